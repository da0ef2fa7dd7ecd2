"""The A/B switches select older code paths of the same arithmetic: with a switch set, the results must not change by a bit.

The switches are read once per process, so every setting runs in a child process that writes its outputs to a file; the parent
computes the same calls with the defaults and compares. Covered: the direct output stores of the CTA-pair GEMMs (the default
sends the output through bulk tensor stores), the K split through scratch and tickets (the default exchanges the partials inside a
cluster where every cluster of the launch fits the device) and the conv kernels that gather from global memory (the default stages
halo tiles through the copy engine) and the int8 GEMM over an unpacked weight (the default reads the row-major weight through the copy
engine, the switch permutes it per call and runs the re-layout kernel) and the pair kernels' tile width (the default picks it by shape, the
switches keep 256 columns).
"""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent(
    """
    import sys
    import torch
    sys.path.insert(0, sys.argv[2])
    import feather_ops_b200 as fo
    from feather_ops_b200 import int8_convrot as ic
    from oracle import conv2d as oc
    from oracle import scaled_mm as osm

    dev = torch.device("cuda", 0)
    out = {}
    # the CTA-pair kernel, and its K split with two and three splits, where the tile's pairs form one cluster and exchange their
    # partials through distributed shared memory unless the switch sends them through scratch and tickets
    for m, n, k in ((600, 2304, 1536), (4096, 1024, 512), (512, 4096, 4096), (256, 5120, 5120), (300, 2048, 6144), (516, 2560, 4096)):
        a, packed, scale, bias = (t.to(dev) for t in osm.make_inputs(m, n, k, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, seed=m + n))
        out[f"smm{m}"] = fo.scaled_mm_hip(a, packed, scale, bias, torch.bfloat16).cpu()
    gen = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn((520, 1280), device=dev, generator=gen).to(torch.bfloat16)
    g = torch.randn((520, 768), device=dev, generator=gen).to(torch.bfloat16)
    w = (torch.randn((768, 1280), device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    wq, ws = ic.quantize_convrot_weight(w)
    packed8 = ic.prepack_int8_weight(wq)
    out["i8f"] = ic.convrot_int8_linear(x, packed8, ws, None, torch.bfloat16, weight_packed=True).cpu()
    out["i8b"] = ic.convrot_int8_dgrad(g, packed8, ws, torch.bfloat16, rotate_activation=False, weight_packed=True).cpu()
    # the unpacked weight: straight through the copy engine, or (switched) permuted per call and through the re-layout kernel
    out["i8f_plain"] = ic.convrot_int8_linear(x, wq, ws, None, torch.bfloat16).cpu()
    out["i8b_plain"] = ic.convrot_int8_dgrad(g, wq, ws, torch.bfloat16, rotate_activation=False).cpu()
    for c_out, hw in ((272, 40), (96, 264)):
        xc, wc, bc = oc.make_inputs(2, 24, c_out, 9, hw, torch.bfloat16, seed=c_out)
        out[f"conv{c_out}"] = fo.conv3x3_prepacked(xc.to(dev), fo.prepack_conv2d_weight_3x3(wc.to(dev)), bc.to(dev)).cpu()
    torch.cuda.synchronize()
    torch.save(out, sys.argv[1])
    """
)


CHILD_SCALED_MM_PAIR = textwrap.dedent(
    """
    import sys
    import torch
    sys.path.insert(0, sys.argv[2])
    import feather_ops_b200  # noqa: F401
    from oracle import scaled_mm as osm

    dev = torch.device("cuda", 0)
    out = {}
    # the CTA-pair kernel without a K split (256-wide tile tuple, more than 128 rows): ragged in every axis, one and several rounds of tiles
    for m, n, k in ((300, 272, 272), (2048, 3072, 512), (1100, 12288, 256), (4112, 1536, 1024), (516, 2576, 4096)):
        a, packed, scale, bias = (t.to(dev) for t in osm.make_inputs(m, n, k, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, seed=m + n))
        c = torch.empty((m, n), device=dev, dtype=torch.bfloat16)
        torch.ops.feather_ops.scaled_mm.default(a, packed, scale, bias, c, 1, 8, 4, 8, 2, False)
        out[f"pair{m}"] = c.cpu()
    torch.cuda.synchronize()
    torch.save(out, sys.argv[1])
    """
)


CHILD_INT8_PLAIN = textwrap.dedent(
    """
    import sys
    import torch
    sys.path.insert(0, sys.argv[2])
    from feather_ops_b200 import int8_convrot as ic

    dev = torch.device("cuda", 0)
    out = {}
    gen = torch.Generator(device=dev).manual_seed(11)
    # forward over the unpacked weight: ragged in every axis, one round and several rounds of tiles
    for m, n, k in ((300, 260, 272), (2048, 3072, 1024), (4096, 3072, 512), (700, 648, 4112), (1100, 12288, 256)):
        a = torch.randint(-127, 128, (m, k), device=dev, generator=gen, dtype=torch.int8)
        w = torch.randint(-127, 128, (n, k), device=dev, generator=gen, dtype=torch.int8)
        s = torch.rand(m, device=dev, generator=gen) * 0.01
        ws = torch.rand(n, device=dev, generator=gen) * 0.01
        bias = torch.randn(n, device=dev, generator=gen).to(torch.bfloat16)
        out[f"plain{m}"] = ic.int8_scaled_mm_plain(a, w, s, ws, bias, torch.bfloat16, False).cpu()
        if n % 16 == 0:
            g = torch.randint(-127, 128, (m, n), device=dev, generator=gen, dtype=torch.int8)
            out[f"plain_backward{m}"] = ic.int8_scaled_mm_plain(g, w, s, None, None, torch.bfloat16, True).cpu()
    torch.cuda.synchronize()
    torch.save(out, sys.argv[1])
    """
)


def _run(tmp_path, name, env, child=CHILD):
    target = tmp_path / f"{name}.pt"
    full_env = dict(os.environ)
    full_env.update(env)
    done = subprocess.run([sys.executable, "-c", child, str(target), ROOT], env=full_env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    return torch.load(target, weights_only=True)


def test_switched_paths_give_the_same_bits(cuda_device, tmp_path):
    default = _run(tmp_path, "default", {})
    switched = _run(tmp_path, "switched", {"FEATHER_SCALED_MM_BULK_OUT_OFF": "1", "FEATHER_INT8_BULK_OUT_OFF": "1", "FEATHER_CONV_STAGING_OFF": "1",
                                           "FEATHER_INT8_PDL_OFF": "1", "FEATHER_SCALED_MM_CLUSTER_REDUCE_OFF": "1", "FEATHER_INT8_PLAIN_OFF": "1",
                                           "FEATHER_INT8_TILE_WIDTH_OFF": "1", "FEATHER_SCALED_MM_TILE_WIDTH_OFF": "1"})
    assert torch.equal(default["i8f"], default["i8f_plain"]) and torch.equal(default["i8b"], default["i8b_plain"])
    assert set(default) == set(switched)
    for key, value in default.items():
        assert torch.equal(value, switched[key]), key


def test_int8_tile_widths_give_the_same_bits(cuda_device, tmp_path):
    # the products over the unpacked weight pick their tile width by shape (backward: 128, 192 or 256 only, a forced 176 or 208 leaves it at 256);
    # every width adds the same int32 sums
    default = _run(tmp_path, "width_default", {}, CHILD_INT8_PLAIN)
    for name, env in (("width_256", {"FEATHER_INT8_TILE_WIDTH_OFF": "1"}), ("width_176", {"FEATHER_INT8_TILE_WIDTH": "176"}),
                      ("width_208", {"FEATHER_INT8_TILE_WIDTH": "208"}), ("width_192", {"FEATHER_INT8_TILE_WIDTH": "192"})):
        other = _run(tmp_path, name, env, CHILD_INT8_PLAIN)
        assert set(default) == set(other)
        for key, value in default.items():
            assert torch.equal(value, other[key]), (name, key)


def test_scaled_mm_tile_widths_give_the_same_bits(cuda_device, tmp_path):
    # the pair kernel picks its tile width by shape; a tile's columns are accumulated in the same order whatever its width
    default = _run(tmp_path, "smm_width_default", {}, CHILD_SCALED_MM_PAIR)
    for name, env in (("smm_width_256", {"FEATHER_SCALED_MM_TILE_WIDTH_OFF": "1"}), ("smm_width_160", {"FEATHER_SCALED_MM_TILE_WIDTH": "160"})):
        other = _run(tmp_path, name, env, CHILD_SCALED_MM_PAIR)
        assert set(default) == set(other)
        for key, value in default.items():
            assert torch.equal(value, other[key]), (name, key)
