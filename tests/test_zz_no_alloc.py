"""The allocation-free split-K entry point against the caller-scratch one.

`launch_scaled_mm_splitk_static` is for hosts that cannot allocate device memory while they run (all memory
already given to their own arena, an FFI plugin with no device allocator, a callback where allocation is
forbidden): its partials and tickets live in a fixed array inside the library. It must give exactly what
`launch_scaled_mm_splitk` gives with scratch from the caller, call after call, because both run the same
kernel with the same split order. This file sorts last on purpose, so a stop-at-first-failure run has
already been through every other test.
"""

import ctypes

import pytest
import torch

from feather_ops_b200 import _lib
from oracle import scaled_mm as osm
from tests import _cabi


def _static(a, packed, scale, bias, out_dtype, splits):
    m, k = a.shape
    n = packed.shape[1]
    c = _cabi.guarded_empty((m, n), a.device, out_dtype)
    message = ctypes.create_string_buffer(256)
    rc = _lib.load().launch_scaled_mm_splitk_static(
        a.data_ptr(), packed.data_ptr(), None if scale is None else scale.data_ptr(), None if bias is None else bias.data_ptr(), c.data_ptr(),
        m, n, k, int(scale is not None), int(bias is not None), packed.dtype == torch.float8_e5m2, a.dtype == torch.bfloat16,
        out_dtype == torch.bfloat16, splits, torch.cuda.current_stream().cuda_stream, message, len(message),
    )
    return rc, c, message.value.decode()


def test_sizes_beyond_the_built_in_scratch_are_refused_before_any_cuda_call():
    lib = _lib.load()
    message = ctypes.create_string_buffer(256)
    for m, n, k, splits in ((17, 1024, 1024, 2), (4, 16384 + 64, 1024, 2)):
        rc = lib.launch_scaled_mm_splitk_static(None, None, None, None, None, m, n, k, 0, 0, True, True, True, splits, None, message, len(message))
        assert rc == 2 and b"exceeds the built-in scratch" in message.value
    rc = lib.launch_scaled_mm_splitk_static(None, None, None, None, None, 4, 1000, 1024, 0, 0, True, True, True, 2, None, message, len(message))
    assert rc == 1 and b"multiples of 16" in message.value
    assert lib.launch_scaled_mm_splitk_static(None, None, None, None, None, 0, 1024, 1024, 0, 0, True, True, True, 2, None, None, 0) == 0


# Every case asks for more than one K split, so every case runs the kernel that writes partial tiles and draws tickets:
# the scratch inside the library is really used. The last case is the entry point's bound (16 rows, 16384 columns,
# 4 splits): it fills all 4 MiB of partials and all 256 tickets.
@pytest.mark.gpu
@pytest.mark.parametrize("shape,splits", [((16, 496, 8192), 4), ((9, 272, 4096), 4), ((7, 272, 1040), 2), ((1, 12288, 3072), 3), ((16, 16384, 1024), 4)])
def test_two_calls_in_a_row_equal_the_caller_scratch_entry_point(cuda_device, shape, splits):
    m, n, k = shape
    a, packed, scale, bias = (t.to(cuda_device) for t in osm.make_inputs(m, n, k, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, seed=n + k))
    expected, partials, _ = _cabi.scaled_mm_splitk(a, packed, scale, bias, torch.bfloat16, splits)
    assert partials.numel() == splits * m * n  # the caller-scratch call did split K this many ways
    other, _, _ = _cabi.scaled_mm_splitk((a * 2).contiguous(), packed, scale, None, torch.bfloat16, splits)
    # first call, then a different problem through the same scratch, then the first problem again
    rc1, first, msg1 = _static(a, packed, scale, bias, torch.bfloat16, splits)
    rc2, second, msg2 = _static((a * 2).contiguous(), packed, scale, None, torch.bfloat16, splits)
    rc3, third, msg3 = _static(a, packed, scale, bias, torch.bfloat16, splits)
    # a smaller problem afterwards finds the larger one's partials and tickets in the array and must not care
    small = [t.to(cuda_device) for t in osm.make_inputs(3, 144, 512, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, seed=1)]
    rc4, fourth, msg4 = _static(*small, torch.bfloat16, 2)
    torch.cuda.synchronize()
    assert (rc1, rc2, rc3, rc4) == (0, 0, 0, 0), (msg1, msg2, msg3, msg4)
    _cabi.assert_clean("feather_scaled_mm_status")
    # same kernel, same split order: the bits are the same (the tolerance of the other parity tests is not needed)
    assert torch.equal(first, expected)
    assert torch.equal(second, other)
    assert torch.equal(third, expected)
    assert torch.equal(fourth, _cabi.scaled_mm_splitk(*small, torch.bfloat16, 2)[0])
    ref = osm.scaled_mm_f32(a.cpu(), packed.cpu(), scale.cpu(), bias.cpu(), torch.bfloat16, b_prepacked=True)
    rel = ((first.float().cpu() - ref.float()).norm() / ref.float().norm()).item()
    assert rel <= 1e-3


@pytest.mark.gpu
def test_gpu_side_refusal_leaves_the_output_untouched(cuda_device):
    a, packed, scale, _ = (None if t is None else t.to(cuda_device) for t in osm.make_inputs(32, 256, 512, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, with_bias=False))
    c = torch.full((32, 256), 7.0, device=cuda_device, dtype=torch.bfloat16)
    message = ctypes.create_string_buffer(256)
    rc = _lib.load().launch_scaled_mm_splitk_static(
        a.data_ptr(), packed.data_ptr(), scale.data_ptr(), None, c.data_ptr(), 32, 256, 512, 1, 0, True, True, True, 2,
        torch.cuda.current_stream().cuda_stream, message, len(message),
    )
    torch.cuda.synchronize()
    assert rc == 2 and b"use launch_scaled_mm_splitk" in message.value
    assert bool((c == 7.0).all().item())  # nothing was launched
