"""Oracle for `scaled_mm`: `C = cast(cast((A @ upcast(B)) * scale) + bias)`. Test infrastructure only."""

import torch

FP8_DTYPES = (torch.float8_e5m2, torch.float8_e4m3fn)


def prepack_b(b: torch.Tensor) -> torch.Tensor:
    """`[K, N]` fp8 -> `[K_pad/16, N, 16]` with K zero padded to a multiple of 128.

    Restates `prepack_b_for_scaled_mm`, reference feather_ops/scaled_mm.py:137-150.
    """
    k, n = b.shape
    k_pad = (k + 127) // 128 * 128
    raw = torch.zeros((k_pad, n), dtype=torch.uint8)
    raw[:k] = b.view(torch.uint8)
    return raw.reshape(k_pad // 16, 16, n).transpose(1, 2).contiguous().view(b.dtype)


def unpack_b(b_prepacked: torch.Tensor, k: int) -> torch.Tensor:
    """Inverse of `prepack_b` for the first `k` rows (reference feather_ops/naive.py:13-16)."""
    slabs, n, _ = b_prepacked.shape
    raw = b_prepacked.view(torch.uint8).permute(0, 2, 1).reshape(slabs * 16, n)[:k]
    return raw.contiguous().view(b_prepacked.dtype)


def scaled_mm_naive(a, b, scale, bias, out_dtype, b_prepacked=False):
    """The reference's own CPU path, line by line (feather_ops/naive.py:4-41, `bias_dim=1`).

    Both operands are cast to fp16 and multiplied with an fp16 result, the scale is applied in fp32,
    the result is cast to `out_dtype` and the bias is added in `out_dtype`. The fp16 product
    overflows when the weight codes are large (per-tensor scale = absmax / 57344), which is why
    `scaled_mm_f32` exists.
    """
    if b_prepacked:
        b = unpack_b(b, a.shape[1])
    c = a.to(torch.float16) @ b.to(torch.float16)
    if scale is not None:
        c = c.to(torch.float32) * scale.to(torch.float32)
    c = c.to(out_dtype)
    if bias is not None:
        c = c + bias.to(out_dtype)[None, :]
    return c


def scaled_mm_f32(a, b, scale, bias, out_dtype, b_prepacked=False, a_via_fp16=False):
    """The reference kernel's arithmetic with an fp32 accumulator (csrc/hip_kernel.cu:513, 539, 561-566).

    `acc = sum_k A[m,k] * up(B[k,n])` in fp32 (the sum is taken in fp64 and rounded once, which is within
    half an ulp of any fp32 summation order), `r = cast(acc * scale)`, `out = cast(r + bias)` with both
    casts round-to-nearest-even. `a_via_fp16` rounds a bf16 activation to fp16 first, which is what the
    reference kernel does while staging (csrc/hip_kernel.cu:80-85, 264-271). The B200 kernel keeps it in bf16.
    """
    if b_prepacked:
        b = unpack_b(b, a.shape[1])
    a32 = (a.to(torch.float16) if a_via_fp16 else a).to(torch.float64)
    acc = (a32 @ b.to(torch.float32).to(torch.float64)).to(torch.float32)
    if scale is not None:
        acc = acc * scale.to(torch.float32)
    c = acc.to(out_dtype)
    if bias is not None:
        c = (c.to(torch.float32) + bias.to(out_dtype).to(torch.float32)[None, :]).to(out_dtype)
    return c


def make_inputs(m, n, k, a_dtype, b_dtype, out_dtype, seed=0, with_scale=True, with_bias=True, weight_std=None):
    """Seeded CPU inputs. `weight_std=None` is the reference tests' distribution (`randn` cast to fp8,
    tests/test_scaled_mm_hip.py:35-37, 52-56). A float selects the benchmark distribution: `N(0, std)`
    weights quantized with a per-tensor scale of `absmax / 57344` (e5m2) or `absmax / 448` (e4m3)."""
    gen = torch.Generator().manual_seed(seed)
    a = torch.randn((m, k), generator=gen, dtype=torch.float32).to(a_dtype)
    w = torch.randn((k, n), generator=gen, dtype=torch.float32)
    if weight_std is None:
        b = w.to(b_dtype)
        scale = torch.tensor(2.34, dtype=torch.float32) if with_scale else None
    else:
        w = w * weight_std
        top = 57344.0 if b_dtype == torch.float8_e5m2 else 448.0
        scale = (w.abs().max() / top).to(torch.float32)
        b = (w / scale).to(b_dtype)
    bias = torch.randn((n,), generator=gen, dtype=torch.float32).to(out_dtype) if with_bias else None
    return a, prepack_b(b), scale, bias
