"""The N-sharded variant on two GPUs: real kernel, NCCL all-gather over NVLink, against the single-GPU result.

Runs only where two CUDA devices are visible. Each rank is a child process that owns one GPU, multiplies the
full activation by its own column slab of the weight and all-gathers the output; every variant (blocking,
pipelined in row chunks, slab layout in place) must equal, bit for bit, what one GPU computes with the full
weight: a column's value does not depend on which slab it was computed in.
"""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import feather_ops_b200 as fo
        from feather_ops_b200 import _lib, shard
        from oracle import scaled_mm as osm

        verdicts = {}
        for m, n, k in ((64, 1024, 512), (1000, 2048, 1040), (4096, 3072, 3072)):
            a, packed, scale, bias = (t.to(device) for t in osm.make_inputs(m, n, k, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, seed=m + n))
            full = fo.scaled_mm_hip(a, packed, scale, bias, torch.bfloat16)
            start, stop = shard.token_shard(m, rank, world)
            rows = shard.scaled_mm_token_sharded(a, packed, scale, bias, torch.bfloat16, fo.scaled_mm_hip)
            ok = torch.equal(rows, fo.scaled_mm_hip(a[start:stop].contiguous(), packed, scale, bias, torch.bfloat16))
            slab, bias_slab = shard.weight_column_shard(packed, rank, world, bias)
            # within the tolerance of the parity tests of the single-GPU path: a slab is a narrower problem, so the launcher
            # may pick another tile or kernel for it, and then the fp32 sums are taken in another order
            def close(x):
                return ((x.float() - full.float()).norm() / full.float().norm()).item() <= 1e-3

            blocking = shard.scaled_mm_n_sharded(a, slab, scale, bias_slab, torch.bfloat16)
            ok = ok and blocking.shape == (m, n) and close(blocking)
            for chunks in (4, 7):
                piped = shard.scaled_mm_n_sharded(a, slab, scale, bias_slab, torch.bfloat16, chunks=chunks)
                ok = ok and close(piped)
            # same rows per launch as the blocking variant: the same kernel computed it, so the bits are the same
            slabs = shard.scaled_mm_n_sharded(a, slab, scale, bias_slab, torch.bfloat16, layout="slabs")
            ok = ok and slabs.shape == (world, m, n // world) and torch.equal(slabs.permute(1, 0, 2).reshape(m, n), blocking)
            slabs = shard.scaled_mm_n_sharded(a, slab, scale, bias_slab, torch.bfloat16, chunks=4, layout="slabs")
            ok = ok and close(slabs.permute(1, 0, 2).reshape(m, n))
            # every rank holds the same gathered result
            digest = blocking.float().sum().reshape(1)
            both = [torch.empty_like(digest) for _ in range(world)]
            dist.all_gather(both, digest)
            ok = ok and all(torch.equal(both[0], other) for other in both)
            verdicts[(m, n, k)] = bool(ok)
        verdicts["status"] = _lib.read_status("feather_scaled_mm_status")
        results[rank] = verdicts
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two CUDA devices")
def test_n_sharded_all_gather_on_two_gpus_equals_one_gpu():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    results = dict(results)
    assert set(results) == {0, 1}
    for rank, verdicts in results.items():
        assert verdicts.pop("status") == (0, 0), rank
        assert all(verdicts.values()), (rank, verdicts)


def test_interleave_slabs_kernel_equals_the_permute(cuda_device):
    import feather_ops_b200  # noqa: F401
    from feather_ops_b200 import shard

    for world, rows, width, dtype in ((2, 7, 16, torch.bfloat16), (8, 1000, 1536, torch.bfloat16), (3, 129, 48, torch.float16), (4, 0, 64, torch.bfloat16)):
        slabs = torch.randn((world, rows, width), device=cuda_device).to(dtype)
        out = torch.full((rows, world * width), 3.0, device=cuda_device, dtype=dtype)
        shard._interleave(slabs, out)
        assert torch.equal(out, slabs.permute(1, 0, 2).reshape(rows, world * width))


def test_sm_margin_shrinks_the_grid_and_keeps_the_result(cuda_device):
    import feather_ops_b200 as fo
    from feather_ops_b200 import _lib
    from oracle import scaled_mm as osm

    a, packed, scale, bias = (t.to(cuda_device) for t in osm.make_inputs(1500, 1024, 512, torch.bfloat16, torch.float8_e5m2, torch.bfloat16))
    full = fo.scaled_mm_hip(a, packed, scale, bias, torch.bfloat16)
    lib = _lib.load()
    assert lib.feather_scaled_mm_set_sm_margin(40) == 0
    try:
        for tile in ((1, 8, 4, 8, 2, 0), (2, 2, 2, 4, 4, 0)):   # the CTA-pair kernel and the one-CTA kernel
            assert torch.equal(fo.scaled_mm_hip(a, packed, scale, bias, torch.bfloat16, tile=tile), fo.scaled_mm_hip(a, packed, scale, bias, torch.bfloat16, tile=tile))
        assert torch.equal(fo.scaled_mm_hip(a, packed, scale, bias, torch.bfloat16), full)   # which SM computes a tile does not change its value
    finally:
        assert lib.feather_scaled_mm_set_sm_margin(0) == 40
    assert _lib.read_status("feather_scaled_mm_status") == (0, 0)
