"""The multi-GPU story on CPU: two gloo ranks shard experts / columns, compute their part with the oracle, gather,
and the result equals the unsharded oracle. No collective sits on the data path; the gather is only for checking."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from deep_gemm.testing import sharding


def test_expert_and_column_ranges_partition_exactly():
    for n, world in ((8, 2), (32, 8), (7, 4), (3, 8)):
        ranges = [sharding.expert_range(n, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    cols = [sharding.column_range(2112, 4, r) for r in range(4)]
    assert cols[0][0] == 0 and cols[-1][1] == 2112 and all(c[0] % 8 == 0 for c in cols)
    assert all(a[1] == b[0] for a, b in zip(cols, cols[1:]))


def test_balanced_expert_ranges_partition_and_balance():
    import random
    random.seed(1234)
    sizes = [int(random.uniform(0.7, 1.3) * 8192) for _ in range(32)]
    for world in (1, 2, 4, 8):
        ranges = sharding.balanced_expert_ranges(sizes, world)
        assert len(ranges) == world and ranges[0][0] == 0 and ranges[-1][1] == 32
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        assert all(e > b for b, e in ranges)                         # nobody idles with 32 experts
        loads = [sum(sizes[b:e]) for b, e in ranges]
        even = [sum(sizes[b:e]) for b, e in (sharding.expert_range(32, world, r) for r in range(world))]
        assert max(loads) <= max(even)                                # never worse than equal counts
    # more ranks than experts, and an empty problem
    assert sharding.balanced_expert_ranges([100, 200], 4)[:2] == [(0, 1), (1, 2)]
    assert sharding.balanced_expert_ranges([100, 200], 4)[2:] == [(2, 2), (2, 2)]
    assert sharding.balanced_expert_ranges([], 2) == [(0, 0), (0, 0)]


def test_local_psum_layout_matches_global_rows():
    sizes = [300, 0, 513, 255, 256, 1, 700, 90]
    total, psum = sharding.psum_from_sizes(sizes)
    assert (total, psum) == oracle.make_psum_layout(sizes, 256)
    covered = 0
    for rank in range(4):
        local = sharding.shard_psum_layout(sizes, 4, rank)
        assert local['row_begin'] == covered and local['global_rows'] == total
        b, e = local['experts']
        assert local['psum'] == oracle.make_psum_layout(sizes[b:e], 256)[1]
        covered += local['rows']
    assert covered == total


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result_path: str) -> None:
    os.environ['MASTER_ADDR'], os.environ['MASTER_PORT'] = '127.0.0.1', str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                      # every rank builds the same global problem
        sizes, n, k = [130, 40, 0, 257], 48, 96
        total, psum = oracle.make_psum_layout(sizes, 256)
        a = torch.randn(total, k).to(torch.float8_e4m3fn).float()
        b = torch.randn(len(sizes), n, k).to(torch.float8_e4m3fn).float()
        for span in oracle.psum_padding_spans(psum, 256):
            a[span] = 0
        full = oracle.m_grouped_psum_ref(a, b, psum, torch.float32)

        local = sharding.shard_psum_layout(sizes, world, rank)
        e0, e1 = local['experts']
        rows = slice(local['row_begin'], local['row_begin'] + local['rows'])
        mine = oracle.m_grouped_psum_ref(a[rows], b[e0:e1], local['psum'], torch.float32)
        # grouped: gather row blocks (padded to the largest block)
        sizes_t = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(sizes_t, torch.tensor([mine.size(0)]))
        pad = max(int(t.item()) for t in sizes_t)
        chunk = torch.zeros(pad, n)
        chunk[:mine.size(0)] = mine
        chunks = [torch.zeros(pad, n) for _ in range(world)]
        dist.all_gather(chunks, chunk)
        gathered = torch.cat([c[:int(t.item())] for c, t in zip(chunks, sizes_t)])
        ok_grouped = torch.equal(gathered, full)

        # dense: each rank owns a slab of columns
        d_full = oracle.gemm_ref(a[:64], b[0], torch.float32)
        c0, c1 = sharding.column_range(n, world, rank)
        slab = oracle.gemm_ref(a[:64], b[0][c0:c1], torch.float32)
        slabs = [torch.zeros(64, sharding.column_range(n, world, r)[1] - sharding.column_range(n, world, r)[0])
                 for r in range(world)]
        dist.all_gather(slabs, slab) if len({s.shape for s in slabs}) == 1 else None
        ok_dense = torch.equal(torch.cat(slabs, dim=1), d_full) if len({s.shape for s in slabs}) == 1 else \
            torch.equal(slab, d_full[:, c0:c1])
        if rank == 0:
            with open(result_path, 'w') as f:
                f.write(f'{int(ok_grouped)} {int(ok_dense)}')
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_result(tmp_path):
    result = tmp_path / 'result.txt'
    mp.spawn(_worker, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    assert result.read_text() == '1 1'
