"""The bounded device waits: a wait that nothing satisfies gives up, records where, and the kernel ends normally.

Every tcgen05 kernel of the library waits on barriers through one helper with a limit (about two seconds of SM
clocks); a healthy launch never reaches the limit, so the give-up path gets a launch of its own here: a one-CTA
kernel whose first warp waits, with a limit of a tenth of a second, on a barrier that nothing arrives on. Nothing
traps, faults or hangs; the context stays usable, which the test checks by running a real kernel afterwards.
"""

import ctypes

import pytest
import torch

from feather_ops_b200 import _lib
from oracle import scaled_mm as osm
from tests import _cabi

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_recorded_and_the_context_survives(cuda_device):
    lib = _lib.load()
    scratch = torch.zeros(4, device=cuda_device, dtype=torch.int32)
    out = (ctypes.c_uint32 * 5)()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    rc = lib.feather_selftest_wait_runs_out(200_000_000, scratch.data_ptr(), out, torch.cuda.current_stream().cuda_stream)
    stop.record()
    torch.cuda.synchronize()
    assert rc == 0
    site, tag = out[0] & 0xFF, out[0] >> 8
    assert (site, tag, out[1]) == (2, 5, 0)       # the first waiter's site and tag, block 0
    assert out[2] == 0 and out[3] == 1             # its wait did not complete; the CTA's abort flag is up
    assert out[4] == 0                             # the second waiter left through the abort flag, long before its own limit
    assert 20.0 < start.elapsed_time(stop) < 2000.0  # about 0.1 s of SM clocks, not the second waiter's 6.4 s
    # the library's own status words are untouched and the context still runs kernels
    a, packed, scale, bias = osm.make_inputs(200, 272, 304, torch.bfloat16, torch.float8_e5m2, torch.bfloat16)
    got = _cabi.scaled_mm(a.to(cuda_device), packed.to(cuda_device), scale.to(cuda_device), bias.to(cuda_device), torch.bfloat16)
    _cabi.assert_clean("feather_scaled_mm_status")
    ref = osm.scaled_mm_f32(a, packed, scale, bias, torch.bfloat16, b_prepacked=True)
    assert ((got.float().cpu() - ref.float()).norm() / ref.float().norm()).item() <= 1e-3
