"""Oracle for the int8 ConvRot path (quantizer, weight recipe, int8 GEMM). Test infrastructure only."""

import torch

GROUP = 256
_H4 = ((1, 1, 1, -1), (1, 1, -1, 1), (1, -1, 1, 1), (-1, 1, 1, 1))


def build_hadamard(size: int = GROUP, dtype=torch.float32) -> torch.Tensor:
    """Normalized regular Hadamard `h4^(x)n / sqrt(size)` (reference feather_ops/int8_convrot.py:231-252)."""
    n = size
    while n > 1 and n % 4 == 0:
        n //= 4
    if n != 1:
        raise ValueError(f"the regular Hadamard size must be a power of four, got {size}")
    h4 = torch.tensor(_H4, dtype=dtype)
    h = h4
    while h.shape[0] < size:
        h = torch.kron(h, h4)
    return h / (size**0.5)


def rotate(x: torch.Tensor, hadamard: torch.Tensor, group: int = GROUP) -> torch.Tensor:
    """Group-wise `x @ H^T` in x's dtype (reference feather_ops/int8_convrot.py:255-262)."""
    k = x.shape[-1]
    if k % group:
        raise ValueError(f"last axis {k} is not divisible by the group size {group}")
    y = torch.matmul(x.reshape(*x.shape[:-1], k // group, group), hadamard.T.to(x.dtype))
    return y.reshape(x.shape)


def quantize_rowwise_int8(x: torch.Tensor, scale=None):
    """`scale = absmax / 127` (floor 1e-30), `q = clamp(round(x / scale), -127, 127)`
    (reference feather_ops/int8_convrot.py:265-282)."""
    if scale is None:
        scale = (x.abs().amax(dim=-1).float() / 127.0).clamp(min=1e-30)
    elif isinstance(scale, torch.Tensor):
        scale = scale.reshape(-1).to(torch.float32)
    else:
        scale = torch.tensor(scale, dtype=torch.float32)
    q = torch.clamp(torch.round(x.float() / scale.reshape(-1, *([1] * (x.ndim - 1)))), -127.0, 127.0)
    return q.to(torch.int8), scale


def quantize_convrot_weight(weight: torch.Tensor, rotate_dtype=None):
    """Offline weight recipe: matmul rotation in the weight's dtype, then per-row int8
    (reference feather_ops/int8_convrot.py:285-301)."""
    h = build_hadamard(GROUP, torch.float32)
    return quantize_rowwise_int8(rotate(weight.to(rotate_dtype or weight.dtype), h))


def prepack_int8_weight(weight: torch.Tensor) -> torch.Tensor:
    """`[N, K]` -> `[K/4, N/4, 4, 4]` micro-tiles (reference feather_ops/int8_convrot.py:85-92)."""
    n, k = weight.shape
    return weight.reshape(n // 4, 4, k // 4, 4).permute(2, 0, 1, 3).contiguous()


def unpack_int8_weight(prepacked: torch.Tensor) -> torch.Tensor:
    """Inverse permutation (reference feather_ops/int8_convrot.py:95-100)."""
    k4, n4, _, _ = prepacked.shape
    return prepacked.permute(1, 2, 0, 3).reshape(n4 * 4, k4 * 4)


def _butterfly(members, digit_of_output):
    """`((a0 + a1) + a2) + a3 - 2 * a[3 - d]` in fp32, for each output digit d (a list of 4 tensors)."""
    a0, a1, a2, a3 = members
    total = ((a0 + a1) + a2) + a3
    return [total - 2.0 * members[3 - d] for d in digit_of_output]


def hadamard256_radix4(v: torch.Tensor) -> torch.Tensor:
    """The kernel's rotation: four radix-4 stages over the base-4 digits of the index, lowest first,
    unnormalized, every operation in fp32 in this exact order
    (reference csrc/hip_kernel_int8.cu:646-704, `radix4_wave`). `v`: `[..., 256]` float32."""
    assert v.dtype == torch.float32 and v.shape[-1] == GROUP
    lead = v.shape[:-1]
    for stage in range(4):
        stride = 4**stage
        # index = hi * (4 * stride) + d * stride + lo
        x = v.reshape(*lead, GROUP // (4 * stride), 4, stride)
        members = [x[..., j, :] for j in range(4)]
        outs = _butterfly(members, range(4))
        v = torch.stack(outs, dim=-2).reshape(*lead, GROUP)
    return v


def convrot_quantize(x: torch.Tensor, rotate_flag: bool = True, col_scale=None):
    """Restatement of `convrot_quantize_kernel` (reference csrc/hip_kernel_int8.cu:712-714, 740-765, 801-864):
    fp32 radix-4 rotation, one rounding to the input dtype, row absmax, `divisor = max(amax / 127, 1e-30)`,
    `q = clamp(rint(v * (1 / divisor)), -127, 127)`, `scale = divisor / 16` when rotating else `divisor`.
    Without rotation an optional per-column multiplier is applied and rounded to the input dtype first."""
    m, k = x.shape
    if k % GROUP:
        raise ValueError("the contraction axis must be a multiple of the ConvRot group size (256)")
    v = x.to(torch.float32)
    if not rotate_flag and col_scale is not None:
        v = (v * col_scale.to(torch.float32).reshape(1, k)).to(x.dtype).to(torch.float32)
    if rotate_flag:
        v = hadamard256_radix4(v.reshape(m, k // GROUP, GROUP)).reshape(m, k)
    v = v.to(x.dtype).to(torch.float32)
    amax = v.abs().amax(dim=1) if m > 0 else torch.zeros(0)
    divisor = torch.clamp(amax / torch.tensor(127.0, dtype=torch.float32), min=1e-30)
    inv = torch.tensor(1.0, dtype=torch.float32) / divisor
    q = torch.clamp(torch.round(v * inv[:, None]), -127.0, 127.0).to(torch.int8)
    scale = divisor * 0.0625 if rotate_flag else divisor
    return q, scale


def int8_scaled_mm(a, weight_nk, a_scale, w_scale=None, bias=None, out_dtype=torch.bfloat16, transposed_b=False):
    """fp64 dequantized product rounded once to `out_dtype` (reference tests/test_int8_convrot.py:52-62).
    `weight_nk` is the unpacked `[N, K]` int8 weight. Forward contracts K, backward contracts N."""
    w = weight_nk.double()
    acc = a.double() @ (w if transposed_b else w.T)
    out = acc * a_scale.double().reshape(-1, 1)
    if not transposed_b:
        if w_scale is not None:
            out = out * w_scale.double().reshape(1, -1)
        if bias is not None:
            out = out + bias.double().reshape(1, -1)
    return out.to(out_dtype)


def int8_accumulators(a, weight_nk, transposed_b=False):
    """Exact int32 accumulators (computed in int64)."""
    w = weight_nk.to(torch.int64)
    return a.to(torch.int64) @ (w if transposed_b else w.T)


def make_activation(m, k, dtype, seed=0, outlier_fraction=0.01, outlier_gain=20.0):
    """`N(0, 1)` activations with a fraction of the columns scaled up (the benchmark's outlier channels)."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn((m, k), generator=gen, dtype=torch.float32)
    n_out = int(round(k * outlier_fraction))
    if n_out > 0:
        cols = torch.randperm(k, generator=gen)[:n_out]
        x[:, cols] *= outlier_gain
    return x.to(dtype)


def make_weight(n, k, dtype, seed=1, std=0.02):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn((n, k), generator=gen, dtype=torch.float32) * std).to(dtype)
