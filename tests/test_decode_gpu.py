"""Split-K decode, LSE merge, paged-KV decode and the FP32 short-sequence kernel against the oracle.

Modelled on the reference's tests/test_decode.py, tests/test_paged.py, tests/test_tiny.py, tests/test_gqa.py.
"""
import ctypes as C
import math

import pytest
import torch

from helpers import O_TOL, TINY_TOL, assert_close_o, max_abs, seeded
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("sq", [1, 4])
@pytest.mark.parametrize("sk", [128, 1000, 4096, 16384])
def test_decode(dtype, head_dim, sq, sk):
    import fa_b200

    q = seeded(1, 2, 8, sq, head_dim, dtype=dtype)
    k = seeded(2, 2, 8, sk, head_dim, dtype=dtype)
    v = seeded(3, 2, 8, sk, head_dim, dtype=dtype)
    out = fa_b200.flash_attention_decode(q, k, v)
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu())
    assert_close_o(out, ref, dtype)


@pytest.mark.parametrize("head_dim", [16, 32, 256, 512])
def test_decode_other_head_dims(head_dim):
    import fa_b200

    q, k, v = seeded(1, 1, 4, 2, head_dim), seeded(2, 1, 2, 700, head_dim), seeded(3, 1, 2, 700, head_dim)
    out = fa_b200.flash_attention_decode(q, k, v)
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu())
    assert_close_o(out, ref, torch.float16)


def test_decode_gqa_long_cache_and_strided_views():
    import fa_b200

    q = seeded(1, 2, 32, 1, 128)
    k = seeded(2, 2, 8192, 8, 128).transpose(1, 2)  # (B, Hkv, Sk, D) view of a (B, Sk, Hkv, D) cache
    v = seeded(3, 2, 8192, 8, 128).transpose(1, 2)
    out = fa_b200.flash_attention_decode(q, k, v, softmax_scale=0.07)
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu(), softmax_scale=0.07)
    assert_close_o(out, ref, torch.float16)


def test_decode_forced_split_counts_agree():
    from fa_b200 import interface

    q, k, v = seeded(1, 1, 4, 3, 64), seeded(2, 1, 4, 1000, 64), seeded(3, 1, 4, 1000, 64)
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu())
    for splits in (1, 2, 7, 16, 32):  # 32 leaves some slices empty (LSE = -inf partials)
        out = interface._decode_impl(q, k, v, 0.125, splits)
        assert_close_o(out, ref, torch.float16, f"splits={splits}")


def test_decode_rejects_autograd_and_fp32():
    import fa_b200

    q = seeded(1, 1, 2, 1, 64).requires_grad_(True)
    k = seeded(2, 1, 2, 64, 64)
    with pytest.raises(RuntimeError, match="inference-only"):
        fa_b200.flash_attention_decode(q, k, k)
    with pytest.raises(ValueError, match="unsupported dtype"):
        fa_b200.flash_attention_decode(q.detach().float(), k.float(), k.float())


def test_combine_entry_point():
    from fa_b200 import _lib

    lib = _lib.load()
    S, R, D = 5, 37, 64
    o = seeded(1, S, R, D, dtype=torch.float32)
    lse = seeded(2, S, R, dtype=torch.float32)
    lse[1] = float("-inf")
    lse[:, 3] = float("-inf")  # a row with no contribution at all -> zeros, LSE -inf
    out = torch.empty(R, D, dtype=torch.float16, device="cuda")
    lse_out = torch.empty(R, dtype=torch.float32, device="cuda")
    p = _lib.CombineParams()
    p.out_dtype, p.rows, p.head_dim, p.num_splits = _lib.FA_F16, R, D, S
    p.o_partial, p.o_split_stride, p.o_row_stride = o.data_ptr(), R * D, D
    p.lse_partial, p.lse_split_stride, p.lse_row_stride = lse.data_ptr(), R, 1
    p.out, p.out_row_stride, p.lse_out = out.data_ptr(), D, lse_out.data_ptr()
    _lib.check(lib.fa_combine(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    ro, rl = oracle.combine_ref(o.cpu(), lse.cpu())
    assert max_abs(out, ro) <= 2e-3 and max_abs(lse_out, rl) <= 1e-5
    assert torch.all(out[3] == 0) and torch.isinf(lse_out[3])


# ------------------------------------------------------------------------------------------ paged
def make_paged(B, Hq, Hk, D, bs, contexts, dtype=torch.float16, seed=0, shuffle=True):
    max_blocks = max(1, math.ceil(max(contexts) / bs))
    nb = B * max_blocks
    g = torch.Generator().manual_seed(seed)
    q = seeded(seed + 1, B, Hq, D, dtype=dtype)
    kc = seeded(seed + 2, nb, bs, Hk, D, dtype=dtype)
    vc = seeded(seed + 3, nb, bs, Hk, D, dtype=dtype)
    ids = torch.randperm(nb, generator=g) if shuffle else torch.arange(nb)
    table = ids.to(torch.int32).reshape(B, max_blocks).cuda()
    ctx = torch.tensor(contexts, dtype=torch.int32, device="cuda")
    return q, kc, vc, table, ctx


def check_paged(q, kc, vc, table, ctx, dtype=torch.float16, **kw):
    import fa_b200

    out = fa_b200.flash_attention_decode_paged(q, kc, vc, table, ctx, **kw)
    ref, _ = oracle.paged_ref(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), ctx.cpu(), kw.get("softmax_scale"))
    assert_close_o(out, ref, dtype)
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hk", [(8, 8), (8, 2)])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_paged(dtype, hq, hk, head_dim):
    check_paged(*make_paged(3, hq, hk, head_dim, 16, [100, 63, 16], dtype=dtype, seed=hq + hk + head_dim), dtype=dtype)


def test_paged_zero_context_returns_zeros():
    q, kc, vc, table, ctx = make_paged(2, 4, 4, 64, 16, [0, 40])
    out = check_paged(q, kc, vc, table, ctx)
    assert torch.all(out[0] == 0)


@pytest.mark.parametrize("splits", [1, 3, 7, 32])
def test_paged_forced_splits(splits):
    check_paged(*make_paged(2, 8, 2, 128, 16, [1000, 333], seed=splits), num_splits=splits)


@pytest.mark.parametrize("block_size", [8, 32, 64])
def test_paged_block_sizes(block_size):
    check_paged(*make_paged(2, 4, 4, 64, block_size, [257, 64], seed=block_size))


def test_paged_strided_metadata_invalid_ids_and_clamped_context():
    q, kc, vc, table, ctx = make_paged(3, 8, 2, 64, 16, [200, 90, 48], seed=4)
    wide = torch.zeros(3, table.shape[1] * 2, dtype=torch.int32, device="cuda")
    wide[:, ::2] = table
    ctx_wide = torch.zeros(6, dtype=torch.int32, device="cuda")
    ctx_wide[::2] = ctx
    check_paged(q, kc, vc, wide[:, ::2], ctx_wide[::2])
    bad = table.clone()
    bad[0, 2] = -1                      # never dereferenced, contributes nothing
    bad[1, 0] = kc.shape[0] + 5
    check_paged(q, kc, vc, bad, ctx)
    huge = torch.tensor([10 ** 9, -5, 48], dtype=torch.int32, device="cuda")  # clamped to [0, capacity]
    check_paged(q, kc, vc, table, huge)


def test_paged_long_context_auto_split():
    contexts = [16384, 1, 9000, 4097]
    check_paged(*make_paged(4, 32, 8, 128, 16, contexts, seed=6), max_context_len=16384)


def test_paged_kv_shards_merge_to_whole():
    """Every G-th logical block per shard, merged with the LSE rule, equals the unsharded result."""
    from fa_b200 import interface

    q, kc, vc, table, ctx = make_paged(2, 8, 2, 128, 16, [1500, 700], seed=8)
    whole, _ = oracle.paged_ref(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), ctx.cpu())
    for G in (2, 4):
        parts = [interface._paged_launch(q, kc, vc, table, ctx, 1 / math.sqrt(128), 2, first_block=r, block_step=G,
                                         want_lse=True, out_f32=True) for r in range(G)]
        o, _ = oracle.combine_ref(torch.stack([p[0] for p in parts]).cpu(), torch.stack([p[1] for p in parts]).cpu())
        assert max_abs(o, whole) <= 2e-3


# ------------------------------------------------------------------------------------------ tiny
@pytest.mark.parametrize("seqlen", [1, 6, 19, 32])
@pytest.mark.parametrize("bias_kind", ["none", "fp32", "masked_rows"])
def test_tiny_fp32(seqlen, bias_kind):
    import fa_b200
    from fa_b200 import interface

    q, k, v = (seeded(i + seqlen, 2, 8, seqlen, 128, dtype=torch.float32) for i in (1, 2, 3))
    bias = None
    if bias_kind != "none":
        bias = seeded(9, 1, 8, seqlen, seqlen, dtype=torch.float32)
        if bias_kind == "masked_rows":
            bias[:, :, 0, :] = float("-inf")
    assert interface._can_use_tiny_forward(q, k, v, False, (-1, -1), 0.0, None, 0.0, 128)
    out = fa_b200.flash_attention(q, k, v, bias=bias)
    ref = oracle.tiny_ref(q.cpu(), k.cpu(), v.cpu(), bias=None if bias is None else bias.cpu())
    assert max_abs(out, ref) <= TINY_TOL
    if bias_kind == "masked_rows":
        assert torch.all(out[:, :, 0] == 0)


def test_tiny_transposed_layout():
    import fa_b200

    q, k, v = (seeded(i, 2, 19, 8, 128, dtype=torch.float32).transpose(1, 2) for i in (1, 2, 3))
    out = fa_b200.flash_attention(q, k, v)
    assert max_abs(out, oracle.tiny_ref(q.cpu(), k.cpu(), v.cpu())) <= TINY_TOL


# ------------------------------------------------------------------------------------------ kernel families
@pytest.mark.parametrize("path", [1, 2])  # 1 = TMA + tcgen05 kernel, 2 = CUDA-core kernel
@pytest.mark.parametrize("hq,hk,sq,sk,splits", [(8, 8, 1, 4096, 8), (32, 8, 1, 8192, 6), (8, 2, 4, 1000, 4),
                                                (4, 4, 8, 300, 2), (16, 1, 3, 129, 2), (2, 2, 1, 128, 2)])
def test_decode_both_kernel_families(path, hq, hk, sq, sk, splits):
    from fa_b200 import _lib, interface

    q, k, v = seeded(1, 2, hq, sq, 128), seeded(2, 2, hk, sk, 128), seeded(3, 2, hk, sk, 128)
    out = interface._decode_impl(q, k, v, 0.09, splits, force_path=path)
    assert _lib.load().fa_last_path() == path
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu(), softmax_scale=0.09)
    assert_close_o(out, ref, torch.float16)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hk,sq,sk,splits", [(8, 8, 1, 4096, 8), (32, 8, 1, 8192, 5), (8, 2, 4, 1000, 4),
                                                (4, 4, 8, 300, 2), (16, 1, 3, 129, 2), (2, 2, 1, 128, 3),
                                                (8, 2, 1, 16384, 7)])
def test_decode_head_dim_256_both_kernel_families(path, dtype, hq, hk, sq, sk, splits):
    """Head dim 256 on the tensor-core kernel (one softmax stream, one partial per CTA, any split count >= 2) and on
    the CUDA-core kernel."""
    from fa_b200 import _lib, interface

    q, k, v = (seeded(1, 2, hq, sq, 256, dtype=dtype), seeded(2, 2, hk, sk, 256, dtype=dtype),
               seeded(3, 2, hk, sk, 256, dtype=dtype))
    out = interface._decode_impl(q, k, v, 0.0625, splits, force_path=path)
    assert _lib.load().fa_last_path() == path
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu(), softmax_scale=0.0625)
    assert_close_o(out, ref, dtype)


def test_decode_head_dim_256_public_entry():
    import fa_b200
    from fa_b200 import _lib

    q, k, v = seeded(1, 4, 32, 1, 256), seeded(2, 4, 8, 5000, 256), seeded(3, 4, 8, 5000, 256)
    out = fa_b200.flash_attention_decode(q, k, v)
    assert _lib.load().fa_last_path() == 1
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu(), softmax_scale=1.0 / 16.0)
    assert_close_o(out, ref, torch.float16)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("dtype,head_dim", [(torch.float16, 64), (torch.bfloat16, 128)])
@pytest.mark.parametrize("block_size,contexts", [(16, [1000, 333, 0, 16]), (8, [257, 64, 5, 1]), (64, [700, 64, 65, 1]),
                                                 (128, [900, 128, 129, 0])])
def test_paged_both_kernel_families(path, dtype, head_dim, block_size, contexts):
    from fa_b200 import _lib, interface

    q, kc, vc, table, ctx = make_paged(4, 8, 2, head_dim, block_size, contexts, dtype=dtype, seed=block_size)
    scale = 1.0 / math.sqrt(head_dim)
    out, _ = interface._paged_launch(q, kc, vc, table, ctx, scale, 4, force_path=path)
    assert _lib.load().fa_last_path() == path
    ref, _ = oracle.paged_ref(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), ctx.cpu())
    assert_close_o(out, ref, dtype)


@pytest.mark.parametrize("path", [1, 2])
def test_paged_never_reads_past_the_context_or_bad_pages(path):
    """Cache contents past context_len, and whole pages the table does not legitimately reference, are NaN:
    nothing of them may reach the output."""
    from fa_b200 import interface

    B, Hq, Hk, D, bs = 3, 8, 2, 128, 16
    contexts = [200, 77, 33]
    q, kc, vc, table, ctx = make_paged(B, Hq, Hk, D, bs, contexts, seed=11)
    kc, vc = kc.clone(), vc.clone()
    used = torch.zeros(kc.shape[0], bs, dtype=torch.bool, device="cuda")
    for b, c in enumerate(contexts):
        for pos in range(c):
            used[table[b, pos // bs], pos % bs] = True
    kc[~used] = float("nan")
    vc[~used] = float("nan")
    bad = table.clone()
    bad[0, 3] = -7
    bad[1, 1] = kc.shape[0] + 3
    for tbl in (table, bad):
        out, _ = interface._paged_launch(q, kc, vc, tbl, ctx, 1.0 / math.sqrt(D), 4, force_path=path)
        assert not torch.isnan(out.float()).any()
        kz, vz = torch.nan_to_num(kc, nan=0.0), torch.nan_to_num(vc, nan=0.0)
        ref, _ = oracle.paged_ref(q.cpu(), kz.cpu(), vz.cpu(), tbl.cpu(), ctx.cpu())
        assert_close_o(out, ref, torch.float16)


@pytest.mark.parametrize("path", [1, 2])
def test_paged_kv_shards_both_families(path):
    from fa_b200 import interface

    q, kc, vc, table, ctx = make_paged(2, 8, 2, 128, 16, [1500, 700], seed=8)
    whole, _ = oracle.paged_ref(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), ctx.cpu())
    G = 4
    parts = [interface._paged_launch(q, kc, vc, table, ctx, 1 / math.sqrt(128), 2, first_block=r, block_step=G,
                                     want_lse=True, out_f32=True, force_path=path) for r in range(G)]
    o, _ = oracle.combine_ref(torch.stack([p[0] for p in parts]).cpu(), torch.stack([p[1] for p in parts]).cpu())
    assert max_abs(o, whole) <= 2e-3


# ------------------------------------------------------------------------------------------ merge inside the kernel
@pytest.mark.parametrize("hq,hk,sq,sk,splits", [(8, 8, 1, 2048, 2),      # one CTA per head draws the only ticket
                                                (8, 8, 1, 16384, 36),    # 18 CTAs per head, 36 partials
                                                (32, 8, 4, 4096, 8),     # 16 rows per kv head
                                                (64, 1, 2, 4096, 4),     # 128 rows x 128 x 4 = 64 Ki floats: still inside
                                                (64, 1, 2, 4096, 6)])    # one step larger: the merge kernel
def test_decode_merge_inside_and_outside_the_kernel(hq, hk, sq, sk, splits):
    """Small merges are done by the last CTA of each kv head inside the decode kernel, larger ones by the merge
    kernel; twice in a row, so a ticket word that did not return to zero would show."""
    from fa_b200 import _lib, interface

    q, k, v = seeded(1, 2, hq, sq, 128), seeded(2, 2, hk, sk, 128), seeded(3, 2, hk, sk, 128)
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu(), softmax_scale=0.09)
    for _ in range(2):
        out = interface._decode_impl(q, k, v, 0.09, splits, force_path=1)
        assert _lib.load().fa_last_path() == 1
        assert_close_o(out, ref, torch.float16)


def test_decode_merge_inside_the_kernel_on_two_streams():
    """Calls that overlap on the GPU use different partial buffers and therefore different ticket words."""
    from fa_b200 import interface

    cases = []
    for i, sk in enumerate((8192, 12288)):
        q, k, v = seeded(10 + i, 1, 8, 1, 128), seeded(20 + i, 1, 8, sk, 128), seeded(30 + i, 1, 8, sk, 128)
        ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu(), softmax_scale=0.09)
        cases.append((q, k, v, ref, torch.cuda.Stream()))
    torch.cuda.synchronize()
    outs = [[], []]
    for _ in range(8):
        for i, (q, k, v, ref, stream) in enumerate(cases):
            with torch.cuda.stream(stream):
                outs[i].append(interface._decode_impl(q, k, v, 0.09, 16, force_path=1))
    torch.cuda.synchronize()
    for i, (q, k, v, ref, stream) in enumerate(cases):
        for out in outs[i]:
            assert_close_o(out, ref, torch.float16)


# ---------------------------------------------------------------------------------------------------
# The status path of the tensor-core decode kernels. The failure is made on purpose in the allowed form: the
# library's test hook shortens the poll limit and makes the producer leave one tile out, so a wait on a barrier
# that nothing completes runs out, every role leaves through the kernel's normal exit (TMEM freed), the abandoned
# slice hands in an empty partial and the status word is set. Nothing traps, faults or spins without a bound.
# ---------------------------------------------------------------------------------------------------
def test_decode_lost_wait_sets_the_status_word_and_leaves_the_gpu_usable():
    import fa_b200
    from fa_b200 import _lib, interface

    lib = _lib.load()
    q, k, v = seeded(1, 1, 1, 1, 128), seeded(2, 1, 1, 512, 128), seeded(3, 1, 1, 512, 128)
    ref, _ = oracle.decode_ref(q.cpu(), k.cpu(), v.cpu())
    fa_b200.check_status()
    lib.fa_test_decode_fault(1 << 12, 0)  # one CTA (two splits), tile 0 never arrives
    out = interface._decode_impl(q, k, v, 1.0 / math.sqrt(128), 2, force_path=_lib.FA_PATH_TCGEN05)
    with pytest.raises(RuntimeError, match="wait timeout"):
        fa_b200.check_status()
    assert torch.isfinite(out.float()).all()  # the empty partials merge to finite numbers, never to garbage
    fa_b200.check_status()                    # the word was cleared by the failed check
    # the hook is one-shot and the context is intact: the same call now gives the right answer
    out = interface._decode_impl(q, k, v, 1.0 / math.sqrt(128), 2, force_path=_lib.FA_PATH_TCGEN05)
    assert_close_o(out, ref, torch.float16)


def test_paged_lost_wait_sets_the_status_word():
    import fa_b200
    from fa_b200 import _lib, interface

    lib = _lib.load()
    q, kc, vc, table, ctx = make_paged(1, 8, 2, 128, 16, [400], seed=5)
    fa_b200.check_status()
    lib.fa_test_decode_fault(1 << 12, 0)
    out, _ = interface._paged_launch(q, kc, vc, table, ctx, 1.0 / math.sqrt(128), 2, force_path=_lib.FA_PATH_TCGEN05)
    with pytest.raises(RuntimeError, match="wait timeout"):
        fa_b200.check_status()
    assert torch.isfinite(out.float()).all()
    check_paged(q, kc, vc, table, ctx, num_splits=2)


# ------------------------------------------------------------------------------------------ balanced paged decode
@pytest.mark.parametrize("contexts", [[6237, 3218, 12772, 15003], [16384], [1, 16, 17, 0, 300, 5000, 31, 2048],
                                      [0, 0, 0], [100000, 7]])
def test_paged_balanced_ragged_batches(contexts):
    """One CTA per SM dealt to the sequences by context length (what the public entry point uses when the
    tensor-core kernel applies): ragged, empty, tiny and very long sequences in one batch."""
    q, kc, vc, table, ctx = make_paged(len(contexts), 32, 8, 128, 16, contexts, seed=len(contexts))
    check_paged(q, kc, vc, table, ctx, max_context_len=max(max(contexts), 1))
    check_paged(q, kc, vc, table, ctx)


@pytest.mark.parametrize("slots", [2, 4, 10, 64, 296])
def test_paged_balanced_partial_slot_capacity(slots):
    """The number of partial slots per sequence caps the CTAs a sequence gets; unused slots must not reach the merge
    (the buffers start from NaN here)."""
    from fa_b200 import _lib, interface

    contexts = [3000, 40, 9000]
    q, kc, vc, table, ctx = make_paged(3, 8, 2, 64, 16, contexts, seed=9)
    ref, _ = oracle.paged_ref(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), ctx.cpu(), None)
    torch.empty(3 * 8 * slots * 65 + 4096, device="cuda").fill_(float("nan"))  # poison what the allocator hands out next
    out, _ = interface._paged_launch(q, kc, vc, table, ctx, 1.0 / 8, slots, balance=True,
                                     force_path=_lib.FA_PATH_TCGEN05)
    assert_close_o(out, ref, torch.float16)


def test_paged_balanced_kv_shards_merge_to_whole():
    from fa_b200 import _lib, interface

    contexts = [5000, 333, 12000, 64]
    q, kc, vc, table, ctx = make_paged(4, 32, 8, 128, 16, contexts, seed=21)
    ref, _ = oracle.paged_ref(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), ctx.cpu(), None)
    G = 4
    parts = [interface._paged_launch(q, kc, vc, table, ctx, 1 / math.sqrt(128), 64, first_block=r, block_step=G,
                                     want_lse=True, out_f32=True, balance=True, force_path=_lib.FA_PATH_TCGEN05)
             for r in range(G)]
    o, _ = oracle.combine_ref(torch.stack([p[0] for p in parts]).cpu(), torch.stack([p[1] for p in parts]).cpu())
    assert max_abs(o, ref) <= 2e-3


# ---------------------------------------------------------------------------------------------------
# fa_peer_merge on one GPU: the "peer" buffer is a second local allocation and the peer's partial and flag are put
# into this rank's buffer by the host beforehand, so no kernel waits for another one. The two-GPU form is in
# tests/test_multi_gpu.py.
# ---------------------------------------------------------------------------------------------------
def _peer_merge_setup(rows, head_dim, epoch, deliver_peer):
    import ctypes as C

    from fa_b200 import _lib, interface

    g = torch.Generator().manual_seed(rows + head_dim)
    o = torch.randn(2, rows, head_dim, generator=g)
    lse = torch.randn(2, rows, generator=g) * 2
    lse[1, 3] = float("-inf")      # a shard that saw no key for this row
    slot = -(-(rows * (head_dim + 1)) // 4) * 4

    def buffer():
        return torch.zeros(2 * slot, device="cuda"), torch.zeros(4, dtype=torch.int32, device="cuda")

    mine, my_flags = buffer()
    other, other_flags = buffer()
    for r in (0, 1) if deliver_peer else (0,):
        mine[r * slot:r * slot + rows * head_dim] = o[r].reshape(-1).cuda()
        mine[r * slot + rows * head_dim:r * slot + rows * (head_dim + 1)] = lse[r].cuda()
    if deliver_peer:
        my_flags[1] = epoch
    out = torch.empty(rows, head_dim, dtype=torch.float16, device="cuda")
    lse_out = torch.empty(rows, device="cuda")
    p = _lib.PeerMergeParams()
    p.world, p.rank, p.out_dtype, p.rows, p.head_dim, p.epoch, p.slot_floats = 2, 0, _lib.FA_F16, rows, head_dim, epoch, slot
    p.peer_base[0], p.peer_base[1] = mine.data_ptr(), other.data_ptr()
    p.peer_flags[0], p.peer_flags[1] = my_flags.data_ptr(), other_flags.data_ptr()
    p.out, p.out_row_stride, p.lse_out = out.data_ptr(), head_dim, lse_out.data_ptr()
    p.status = interface._status_word(torch.device("cuda", torch.cuda.current_device())).data_ptr()
    torch.cuda.synchronize()
    _lib.check(_lib.load().fa_peer_merge(C.byref(p), interface._stream(torch.device("cuda", torch.cuda.current_device()))))
    torch.cuda.synchronize()
    return o, lse, out, lse_out, mine, other, other_flags, slot


def test_peer_merge_pushes_this_ranks_slot_and_merges_what_has_arrived():
    rows, head_dim, epoch = 96, 128, 7
    o, lse, out, lse_out, mine, other, other_flags, slot = _peer_merge_setup(rows, head_dim, epoch, deliver_peer=True)
    # this rank's slot went into slot 0 of the peer's buffer, bit for bit, and the peer's flag 0 carries the epoch
    assert torch.equal(other[:slot], mine[:slot])
    assert other_flags.tolist() == [epoch, 0, 0, 0]
    # the merge is the LSE-weighted sum over the two shards
    m = torch.maximum(lse[0], lse[1])
    w = torch.exp(lse - m)
    want = (w[0, :, None] * o[0] + w[1, :, None] * o[1]) / (w[0] + w[1])[:, None]
    assert max_abs(out, want) <= 2e-3
    assert (lse_out.cpu() - (m + torch.log(w[0] + w[1]))).abs().max().item() <= 1e-5


def test_peer_merge_lost_wait_sets_the_status_word():
    """Nobody raises the peer's flag: every merge CTA gives up after its bound (about a second), the status word is set
    and the context stays usable."""
    import fa_b200

    fa_b200.check_status()
    _peer_merge_setup(8, 64, 3, deliver_peer=False)
    with pytest.raises(RuntimeError, match="wait timeout"):
        fa_b200.check_status()
    fa_b200.check_status()
    test_peer_merge_pushes_this_ranks_slot_and_merges_what_has_arrived()
