"""Oracle for the 3x3 stride-1 pad-1 NCHW conv2d. Test infrastructure only."""

import torch
import torch.nn.functional as F


def prepack_conv2d_weight_3x3(weight: torch.Tensor) -> torch.Tensor:
    """`[C_out, C_in, 3, 3]` -> `[ceil(C_in/16) * 18, C_out, 8]`, k order (group, tap, channel % 16), zero padded
    channels (reference feather_ops/conv2d.py:147-164). Written index by index:
    `packed[g * 18 + tap * 2 + half, m, j] = w[m, g * 16 + half * 8 + j, tap // 3, tap % 3]`."""
    c_out, c_in = weight.shape[:2]
    groups = (c_in + 15) // 16
    padded = torch.zeros((c_out, groups * 16, 3, 3), dtype=weight.dtype)
    padded[:, :c_in] = weight
    # [m, g, half, j, tap] -> [g, tap, half, m, j]
    w = padded.reshape(c_out, groups, 2, 8, 9).permute(1, 4, 2, 0, 3)
    return w.reshape(groups * 18, c_out, 8).contiguous()


def conv3x3_fp64(x, weight, bias=None):
    """fp64 `F.conv2d(stride=1, padding=1)`, the reference tests' oracle (tests/test_conv3x3.py:58-59)."""
    return F.conv2d(x.double(), weight.double(), None if bias is None else bias.double(), 1, 1)


def conv3x3(x, weight, bias=None):
    """The kernel's arithmetic: fp32-accumulated products, bias added in fp32, one rounding to the tensor
    dtype (reference csrc/hip_conv2d_3x3.cu:456-460). Computed in fp64 and rounded once."""
    return conv3x3_fp64(x, weight, bias).to(x.dtype)


def make_inputs(b, c_in, c_out, h, w, dtype, seed=0, with_bias=True):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn((b, c_in, h, w), generator=gen, dtype=torch.float32).to(dtype)
    wt = (torch.randn((c_out, c_in, 3, 3), generator=gen, dtype=torch.float32) / (9 * c_in) ** 0.5).to(dtype)
    bias = (torch.randn((c_out,), generator=gen, dtype=torch.float32) * 0.01).to(dtype) if with_bias else None
    return x, wt, bias
