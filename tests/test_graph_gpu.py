"""The entry points take part in CUDA stream capture: a captured forward + backward (with its dependent-launch
edge between the dK/dV and dQ kernels) and a captured decode step replay to the same results as eager calls."""
import math

import pytest
import torch

from helpers import max_abs, seeded

pytestmark = pytest.mark.gpu


def test_forward_backward_replays_from_a_graph():
    from fa_b200 import interface

    B, H, S, D = 2, 4, 512, 128
    q, k, v, dout = (seeded(i, B, H, S, D) for i in (1, 2, 3, 4))
    scale = 1.0 / math.sqrt(D)
    args = (True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    out_e, lse_e = interface._forward(q, k, v, *args)
    grads_e = interface._backward(dout, q, k, v, out_e, lse_e, *args)
    torch.cuda.synchronize()

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up on the capture stream, as torch asks for
        interface._backward(dout, q, k, v, *interface._forward(q, k, v, *args), *args)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_g, lse_g = interface._forward(q, k, v, *args)
        grads_g = interface._backward(dout, q, k, v, out_g, lse_g, *args)
    for t in (out_g, lse_g, *grads_g):
        t.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    assert max_abs(out_g, out_e) == 0.0 and max_abs(lse_g, lse_e) == 0.0
    for got, want in zip(grads_g, grads_e):
        assert max_abs(got, want) == 0.0  # fixed summation order: bit-identical


def test_decode_replays_from_a_graph():
    import fa_b200

    q, k, v = seeded(1, 2, 8, 1, 128), seeded(2, 2, 8, 4096, 128), seeded(3, 2, 8, 4096, 128)
    eager = fa_b200.flash_attention_decode(q, k, v)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fa_b200.flash_attention_decode(q, k, v)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = fa_b200.flash_attention_decode(q, k, v)
    captured.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert max_abs(captured, eager) == 0.0


def test_paged_decode_replays_from_a_graph():
    """Under capture the paged kernel keeps its separate merge kernel (the merge inside the kernel needs a cooperative
    launch); the replayed result equals the eager one up to the different summation order of the two merges."""
    import fa_b200
    from test_decode_gpu import make_paged

    q, kc, vc, table, ctx = make_paged(3, 32, 8, 128, 16, [3000, 40, 1777], seed=21)
    eager = fa_b200.flash_attention_decode_paged(q, kc, vc, table, ctx)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fa_b200.flash_attention_decode_paged(q, kc, vc, table, ctx)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = fa_b200.flash_attention_decode_paged(q, kc, vc, table, ctx)
    for _ in range(3):
        captured.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert max_abs(captured, eager) <= 1e-3
    fa_b200.check_status()
