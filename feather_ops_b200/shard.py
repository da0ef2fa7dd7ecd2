"""Data-parallel sharding of the matmul path over the GPUs of one node (one process per GPU).

The path shards on the token dimension M: every rank multiplies its own rows of A against a replicated
prepacked weight and owns the same rows of C, with no collective. The optional N-sharded variant keeps one
column slab of the weight per rank and all-gathers the output slabs with one NCCL collective. The compute
function is a parameter so the partition logic can be exercised on CPU ranks (gloo) with a stand-in.
"""

from collections.abc import Callable

import torch
import torch.distributed as dist


def token_shard(m_total: int, rank: int, world: int) -> tuple[int, int]:
    """`[start, stop)` rows of rank `rank`: contiguous, balanced to within one row, covering `m_total` exactly."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in [0, {world})")
    base, extra = divmod(m_total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def weight_column_shard(b_prepacked: torch.Tensor, rank: int, world: int, bias: torch.Tensor | None = None):
    """Rank `rank`'s column slab of a `[K_pad/16, N, 16]` prepacked weight (and of the bias). The prepack is
    column-separable, so the slab is a plain slice along dim 1; its width must stay a multiple of 16."""
    n = b_prepacked.shape[1]
    if n % world or (n // world) % 16:
        raise ValueError(f"N={n} does not split into {world} slabs that are multiples of 16 wide")
    width = n // world
    cols = slice(rank * width, (rank + 1) * width)
    return b_prepacked[:, cols].contiguous(), None if bias is None else bias[cols].contiguous()


def scaled_mm_token_sharded(a: torch.Tensor, b_prepacked, scale, bias, out_dtype, matmul: Callable, group=None) -> torch.Tensor:
    """This rank's rows of `C` from the full `a` (every rank holds or can slice the global batch)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    start, stop = token_shard(a.shape[0], rank, world)
    return matmul(a[start:stop].contiguous(), b_prepacked, scale, bias, out_dtype)


def scaled_mm_n_sharded(a: torch.Tensor, b_slab, scale, bias_slab, out_dtype, matmul: Callable, group=None) -> torch.Tensor:
    """Full `C[M, N]` on every rank from per-rank weight slabs: local product, then one all-gather of the
    `[M, N / world]` slabs (`[world, M, N / world]` on the wire, permuted to row-major `[M, N]` afterwards)."""
    world = dist.get_world_size(group)
    local = matmul(a, b_slab, scale, bias_slab, out_dtype).contiguous()
    rows, width = local.shape
    gathered = torch.empty((world * rows, width), device=local.device, dtype=local.dtype)
    dist.all_gather_into_tensor(gathered, local, group=group)
    return gathered.view(world, rows, width).permute(1, 0, 2).reshape(rows, world * width)
