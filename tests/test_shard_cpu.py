"""The multi-GPU partition logic on two CPU ranks (gloo), with the CPU oracle standing in for the kernel."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from feather_ops_b200 import shard
from oracle import scaled_mm as osm


def test_row_chunks_cover_the_rows():
    assert shard.row_chunks(10, 3) == [(0, 4), (4, 7), (7, 10)]
    assert shard.row_chunks(2, 8) == [(0, 1), (1, 2)]
    assert shard.row_chunks(0, 4) == [(0, 0)]


def test_token_shards_cover_the_batch():
    for m in (0, 1, 7, 4096, 65536, 65537):
        for world in (1, 2, 3, 8):
            spans = [shard.token_shard(m, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    with pytest.raises(ValueError):
        shard.token_shard(8, 2, 2)


def test_weight_slabs_are_slices_of_the_prepack():
    _, packed, _, bias = osm.make_inputs(4, 96, 144, torch.bfloat16, torch.float8_e5m2, torch.bfloat16)
    full = osm.unpack_b(packed, 144)
    for rank in range(2):
        slab, bias_slab = shard.weight_column_shard(packed, rank, 2, bias)
        assert torch.equal(osm.unpack_b(slab, 144).view(torch.uint8), full[:, rank * 48 : rank * 48 + 48].contiguous().view(torch.uint8))
        assert torch.equal(bias_slab, bias[rank * 48 : rank * 48 + 48])
    with pytest.raises(ValueError):
        shard.weight_column_shard(packed, 0, 4)  # 24-wide slabs are not multiples of 16


def _oracle_mm(a, b, scale, bias, out_dtype):
    return osm.scaled_mm_f32(a, b, scale, bias, out_dtype, b_prepacked=True)


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a, packed, scale, bias = osm.make_inputs(37, 96, 144, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, seed=5)
        full = _oracle_mm(a, packed, scale, bias, torch.bfloat16)
        mine = shard.scaled_mm_token_sharded(a, packed, scale, bias, torch.bfloat16, _oracle_mm)
        start, stop = shard.token_shard(37, rank, world)
        ok_rows = torch.equal(mine, full[start:stop])
        slab, bias_slab = shard.weight_column_shard(packed, rank, world, bias)
        gathered = shard.scaled_mm_n_sharded(a, slab, scale, bias_slab, torch.bfloat16, _oracle_mm)
        ok_cols = torch.equal(gathered, full)
        # the pipelined variants (row chunks, ragged last chunk) and the slab layout give the same numbers
        for chunks in (3, 64):
            piped = shard.scaled_mm_n_sharded(a, slab, scale, bias_slab, torch.bfloat16, _oracle_mm, chunks=chunks)
            ok_cols = ok_cols and torch.equal(piped, full)
        for chunks in (1, 4):
            slabs = shard.scaled_mm_n_sharded(a, slab, scale, bias_slab, torch.bfloat16, _oracle_mm, chunks=chunks, layout="slabs")
            ok_cols = ok_cols and slabs.shape == (world, 37, 48) and torch.equal(slabs.permute(1, 0, 2).reshape(37, 96), full)
        results[rank] = (ok_rows, ok_cols)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_single_rank_result():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: (True, True), 1: (True, True)}
