"""Data-parallel sharding of the matmul path over the GPUs of one node (one process per GPU).

The path shards on the token dimension M: every rank multiplies its own rows of A against a replicated
prepacked weight and owns the same rows of C, with no collective. The optional N-sharded variant keeps one
column slab of the weight per rank and all-gathers the output slabs over NVLink with NCCL (plain NCCL
collectives on this rank's own buffers; no kernel here reads a peer's memory). The compute function is a
parameter so the partition logic can be exercised on CPU ranks (gloo) with a stand-in.

N-sharded variants, all returning the same numbers:

* `layout="row_major"`, `chunks=1`: local product, one blocking all-gather into `[world, M, N / world]`, one
  permute copy to row-major `[M, N]`.
* `layout="row_major"`, `chunks > 1`: the rows are cut into chunks; the all-gather of chunk i runs on the
  collective's own stream while the compute stream multiplies chunk i + 1 and permutes chunk i - 1. The
  all-gather moves `(world - 1) / world` of the output through every GPU's links and is several times longer
  than the product, so the pipeline hides the product and the copies behind it, not the other way round.
* `layout="slabs"`: the result stays `[world, M, N / world]` (slab g holds columns `[g N / world, (g + 1) N / world)`),
  for callers that can consume it that way. Every rank computes straight into its own slab and the all-gather
  runs in place, so there is no copy at all; with `chunks > 1` each chunk's blocks are gathered into their final
  position.
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


def _kernel_into(a, b_slab, scale, bias_slab, out) -> None:
    """The library's own operator writing into a caller-provided output (tile and split choice included)."""
    from .scaled_mm import _scaled_mm_auto

    _scaled_mm_auto(a, b_slab, scale, bias_slab, out)


def _interleave(gathered: torch.Tensor, out: torch.Tensor) -> None:
    """`out[r, g * width : (g + 1) * width] = gathered[g, r, :]`: the library's copy kernel on CUDA, a strided torch copy elsewhere."""
    world, rows, width = gathered.shape
    if gathered.is_cuda and gathered.dtype in (torch.bfloat16, torch.float16) and width % 8 == 0:
        torch.ops.feather_ops.interleave_slabs.default(gathered, out)
    else:
        out.view(rows, world, width).copy_(gathered.permute(1, 0, 2))


_SIDE_STREAMS: dict = {}


def _side_stream(device: torch.device):
    """One extra stream per device for the copies that run beside the products."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device)
    return _SIDE_STREAMS[key]


class _SmMargin:
    """Leave `sms` SMs free in the persistent scaled_mm kernels while a collective runs beside them (restored on exit).
    A persistent CTA holds its SM's shared memory until the kernel ends, so without free SMs the collective's kernel
    would only start when the product has finished, and nothing would overlap."""

    def __init__(self, sms: int, active: bool) -> None:
        self.sms, self.active, self.previous = sms, active and sms > 0, 0

    def __enter__(self):
        if self.active:
            from . import _lib

            self.previous = _lib.load().feather_scaled_mm_set_sm_margin(self.sms)
        return self

    def __exit__(self, *exc) -> None:
        if self.active:
            from . import _lib

            _lib.load().feather_scaled_mm_set_sm_margin(self.previous)


def row_chunks(rows: int, chunks: int) -> list[tuple[int, int]]:
    """`chunks` contiguous row ranges covering `rows` (fewer when there are fewer rows), balanced to within one row."""
    chunks = max(1, min(chunks, rows)) if rows > 0 else 1
    return [token_shard(rows, i, chunks) for i in range(chunks)]


def scaled_mm_n_sharded(a: torch.Tensor, b_slab, scale, bias_slab, out_dtype, matmul: Callable | None = None, group=None, *, chunks: int = 1,
                        layout: str = "row_major", matmul_into: Callable | None = None, sm_margin: int = 32) -> torch.Tensor:
    """Full `C` on every rank from per-rank weight slabs: local product, then an all-gather of the `[M, N / world]` slabs.

    `matmul(a, b, scale, bias, out_dtype) -> Tensor` or `matmul_into(a, b, scale, bias, out) -> None` computes the local
    product (default: this library's kernel, writing in place). `layout` is `"row_major"` (`[M, N]`) or `"slabs"`
    (`[world, M, N / world]`); `chunks > 1` pipelines the all-gather of one row chunk against the product of the next,
    with `sm_margin` SMs left free by the library's kernel for the collective's kernel to run on.
    """
    if layout not in ("row_major", "slabs"):
        raise ValueError(f"layout must be 'row_major' or 'slabs', got {layout!r}")
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows = a.shape[0]
    width = b_slab.shape[1]
    if matmul is None and matmul_into is None:
        matmul_into = _kernel_into

    def compute(a_rows: torch.Tensor, out: torch.Tensor) -> None:
        if matmul_into is not None:
            matmul_into(a_rows, b_slab, scale, bias_slab, out)
        else:
            out.copy_(matmul(a_rows, b_slab, scale, bias_slab, out_dtype))

    spans = row_chunks(rows, chunks)
    with _SmMargin(sm_margin, a.is_cuda and len(spans) > 1 and matmul is None):
        return _n_sharded(a, compute, spans, world, rank, rows, width, out_dtype, layout, group)


def _n_sharded(a, compute, spans, world, rank, rows, width, out_dtype, layout, group) -> torch.Tensor:
    if layout == "slabs":
        slabs = torch.empty((world, rows, width), device=a.device, dtype=out_dtype)
        if len(spans) == 1:
            # the local product lands in this rank's slab and the all-gather runs in place: no copy anywhere
            compute(a, slabs[rank])
            # NCCL gathers in place when the send buffer is this rank's block of the receive buffer; other backends get a copy
            mine = slabs[rank] if dist.get_backend(group) == "nccl" else slabs[rank].clone()
            dist.all_gather_into_tensor(slabs.view(world * rows, width), mine, group=group)
            return slabs
        works = []
        for start, stop in spans:
            mine = slabs[rank, start:stop]
            compute(a[start:stop], mine)
            # block (g, chunk) of the result is contiguous inside slab g: gather every rank's block into its final place
            send = mine if dist.get_backend(group) == "nccl" else mine.clone()
            works.append(dist.all_gather([slabs[g, start:stop] for g in range(world)], send, group=group, async_op=True))
        for work in works:
            work.wait()
        return slabs

    if len(spans) == 1:
        local = torch.empty((rows, width), device=a.device, dtype=out_dtype)
        compute(a, local)
        gathered = torch.empty((world * rows, width), device=a.device, dtype=out_dtype)
        dist.all_gather_into_tensor(gathered, local, group=group)
        out = torch.empty((rows, world * width), device=a.device, dtype=out_dtype)
        _interleave(gathered.view(world, rows, width), out)
        return out

    out = torch.empty((rows, world * width), device=a.device, dtype=out_dtype)
    pending = None   # (work, gathered chunk, start, stop) of the chunk whose all-gather is in flight
    # The copies into place run on a stream of their own: on the compute stream they would sit between two products and
    # lengthen its chain (product + copy per chunk) past the all-gather's; beside it they use the SMs the margin leaves free.
    on_gpu = a.is_cuda
    main = torch.cuda.current_stream(a.device) if on_gpu else None
    side = _side_stream(a.device) if on_gpu else None
    if on_gpu:
        side.wait_stream(main)   # `out` and the chunks are allocated in the compute stream's order

    def finish(item) -> None:
        work, gathered, start, stop = item
        if on_gpu:
            with torch.cuda.stream(side):
                work.wait()   # the side stream waits for the collective's stream; the host does not block
                _interleave(gathered.view(world, stop - start, width), out[start:stop])
        else:
            work.wait()
            _interleave(gathered.view(world, stop - start, width), out[start:stop])

    # The chunk buffers are allocated on the compute stream, which never waits for a collective here (the side stream
    # does): they stay referenced until the compute stream has joined the side stream, or the allocator could hand a block
    # to the next chunk while the collective still reads it.
    keep = []
    for start, stop in spans:
        local = torch.empty((stop - start, width), device=a.device, dtype=out_dtype)
        compute(a[start:stop], local)
        gathered = torch.empty((world * (stop - start), width), device=a.device, dtype=out_dtype)
        work = dist.all_gather_into_tensor(gathered, local, group=group, async_op=True)
        keep.append((local, gathered))
        if pending is not None:
            finish(pending)   # issued after this chunk's all-gather, so the collective does not wait for the copy
        pending = (work, gathered, start, stop)
    if pending is not None:
        finish(pending)
    if on_gpu:
        main.wait_stream(side)   # the caller's stream sees the whole result, and every collective has finished before it
    del keep
    return out
