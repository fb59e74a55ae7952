"""Two ranks on two GPUs: KV-sharded paged decode against the single-GPU result over NCCL and over peer stores, and
the batch x head partition of the dense path. Skipped when fewer than two GPUs are visible. Ranks are child processes; every rank
joins and leaves the process group between steps, none of them fails on purpose."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    import sys

    import torch.distributed as dist

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "tests"), os.path.join(root, "flash-attention-rdna3_b200")]
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        import fa_b200
        from fa_b200 import distributed as fd
        from helpers import max_abs, seeded
        from oracle import attention_oracle as oracle
        from test_decode_gpu import make_paged

        # every rank builds the same problem on its own GPU; rank r only reads the pages of blocks r, r + world, ...
        q, kc, vc, table, ctx = make_paged(3, 32, 8, 128, 16, [4000, 0, 777], seed=11)
        out = fd.paged_decode_kv_sharded(q, kc, vc, table, ctx, transport="nccl")
        whole = fa_b200.flash_attention_decode_paged(q, kc, vc, table, ctx)
        # the same through peer stores instead of the all-gather: several calls in a row (the two buffer sets and the
        # epochs), then a different query so that a stale slot would show
        push_error, push_diff = None, 0.0
        try:
            for _ in range(5):
                pushed = fd.paged_decode_kv_sharded(q, kc, vc, table, ctx, transport="push")
                push_diff = max(push_diff, max_abs(pushed, out))
            q2 = (q.float() * 0.5 + 0.25).to(q.dtype)
            want2 = fd.paged_decode_kv_sharded(q2, kc, vc, table, ctx, transport="nccl")
            for _ in range(3):
                push_diff = max(push_diff, max_abs(fd.paged_decode_kv_sharded(q2, kc, vc, table, ctx, transport="push"),
                                                   want2))
        except Exception as exc:   # reported to the parent, which fails the test with the reason
            push_error = f"{type(exc).__name__}: {exc}"
        ref, _ = oracle.paged_ref(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), ctx.cpu())
        err_sharded = max_abs(out, ref)
        err_vs_whole = max_abs(out, whole)

        # dense path: ranks take disjoint kv-head slices, nothing is exchanged; gather only to compare
        qd, kd, vd = seeded(1, 2, 8, 300, 64), seeded(2, 2, 4, 300, 64), seeded(3, 2, 4, 300, 64)
        qs, ks, vs = fd.shard_dense_by_heads(qd, kd, vd, world, rank)
        part = fa_b200.flash_attention(qs, ks, vs, causal=True).contiguous()
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        full = fa_b200.flash_attention(qd, kd, vd, causal=True)
        err_dense = max_abs(torch.cat(parts, dim=1), full)
        torch.cuda.synchronize()
        fd.release_peer_buffers()
        fa_b200.check_status(torch.device("cuda", rank))
        results[rank] = (err_sharded, err_vs_whole, err_dense, push_error, push_diff)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_kv_sharded_decode_and_head_partition():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        for rank in range(2):
            err_sharded, err_vs_whole, err_dense, push_error, push_diff = results[rank]
            assert push_error is None, (rank, push_error)
            assert push_diff == 0.0, (rank, push_diff)           # same partials, same merge order: identical
            assert err_sharded <= 2e-3, (rank, err_sharded)      # fp16 output tolerance against the oracle
            assert err_vs_whole <= 2e-3, (rank, err_vs_whole)
            assert err_dense == 0.0, (rank, err_dense)           # same kernels on the same rows: identical
