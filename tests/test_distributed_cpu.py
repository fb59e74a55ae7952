"""World-size-2 gloo tests of the multi-GPU host logic (no GPU): the batch x head partition, and the
KV-sharded paged decode protocol (block-cyclic shards, all-gather of (O, LSE) partials, LSE merge) with the
CUDA kernels replaced by the CPU oracle. A rank that disagrees on the problem must raise on every rank."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_partial(q, kc, vc, table, ctx, scale, rank, world):
    return oracle.paged_ref(q, kc, vc, table, ctx, scale, first_block=rank, block_step=world)


def _oracle_merge(g_o, g_lse, dtype):
    return oracle.combine_ref(g_o, g_lse)[0].to(dtype)


def _worker(rank, world, port, mode, results):
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "flash-attention-rdna3_b200")]
    from fa_b200 import distributed as fd

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        B, Hq, Hk, D, bs, maxb = 3, 4, 2, 32, 8, 10
        q = torch.randn(B, Hq, D, generator=g).half()
        kc = torch.randn(B * maxb, bs, Hk, D, generator=g).half()
        vc = torch.randn(B * maxb, bs, Hk, D, generator=g).half()
        table = torch.randperm(B * maxb, generator=g).to(torch.int32).reshape(B, maxb)
        ctx = torch.tensor([77, 0, 9], dtype=torch.int32)     # one shard of sequence 2 is empty, sequence 1 is empty
        if mode == "merge":
            out = fd.paged_decode_kv_sharded(q, kc, vc, table, ctx, _local_partial=_oracle_partial,
                                             _merge=_oracle_merge)
            whole, _ = oracle.paged_ref(q, kc, vc, table, ctx)
            results[rank] = float((out.float() - whole).abs().max())
        elif mode == "mismatch":
            if rank == 1:
                q = q[:, :2]
            try:
                fd.paged_decode_kv_sharded(q, kc, vc, table, ctx, _local_partial=_oracle_partial,
                                           _merge=_oracle_merge)
                results[rank] = "no error"
            except ValueError as e:
                results[rank] = "ValueError" if "disagree" in str(e) else str(e)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["merge", "mismatch"])
def test_kv_sharded_paged_decode_protocol(mode):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), mode, results), nprocs=world, join=True)
    if mode == "merge":
        assert all(results[r] <= 2e-3 for r in range(world)), dict(results)
    else:
        assert all(results[r] == "ValueError" for r in range(world)), dict(results)


def test_requires_initialised_process_group():
    from fa_b200 import distributed as fd

    q = torch.zeros(1, 2, 16, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="process group"):
        fd.paged_decode_kv_sharded(q, None, None, None, None)


def test_partition_covers_every_group_exactly_once():
    from fa_b200 import distributed as fd

    for batch, heads, world in [(2, 16, 8), (4, 8, 8), (1, 3, 2), (5, 7, 4), (1, 1, 8)]:
        seen = []
        for r in range(world):
            a, b = fd.partition_batch_heads(batch, heads, world, r)
            assert 0 <= a <= b <= batch * heads
            seen += list(range(a, b))
        assert seen == list(range(batch * heads))
        sizes = [fd.partition_batch_heads(batch, heads, world, r) for r in range(world)]
        assert max(b - a for a, b in sizes) - min(b - a for a, b in sizes) <= 1
    with pytest.raises(ValueError):
        fd.partition_batch_heads(2, 2, 2, 2)


def test_head_sliced_views_share_storage():
    from fa_b200 import distributed as fd

    q, k = torch.zeros(2, 32, 4, 8), torch.zeros(2, 8, 6, 8)
    for r in range(4):
        qs, ks, vs = fd.shard_dense_by_heads(q, k, k, 4, r)
        assert qs.shape == (2, 8, 4, 8) and ks.shape == (2, 2, 6, 8)
        assert qs.data_ptr() == q[:, 8 * r:].data_ptr()
    with pytest.raises(ValueError):
        fd.shard_dense_by_heads(q, k, k, 3, 0)
