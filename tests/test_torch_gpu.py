"""torch tensors as kernel arguments: launches go to torch's current stream and can be captured
in a CUDA graph (what a caller does with a launch-bound inner loop)."""

import numpy as np
import pytest

from mytriton_b200 import dot_codegen
from mytriton_b200 import kernels as corpus

pytestmark = pytest.mark.gpu


def test_launches_are_captured_in_a_cuda_graph_and_replay(gpu):
    """A softmax, a tl.dot that fills the GPU's CTA pairs and a small tl.dot that splits K (two
    kernels per call) are recorded on a side stream; replaying the graph on new input contents
    gives what the same launches give eagerly."""
    import torch

    device = torch.device("cuda", 0)
    gen = torch.Generator(device=device).manual_seed(5)
    x = torch.randn(256, 1000, generator=gen, device=device)
    y = torch.empty_like(x)
    a = (torch.randn(512, 2048, generator=gen, device=device) / 45).bfloat16()
    b = torch.randn(2048, 512, generator=gen, device=device).bfloat16()
    c = torch.empty(512, 512, device=device)
    big_a = (torch.randn(2048, 256, generator=gen, device=device) / 16).bfloat16()
    big_b = torch.randn(256, 8192, generator=gen, device=device).bfloat16()
    big_c = torch.empty(2048, 8192, device=device)

    softmax = corpus.softmax_kernel.launcher((256,), x, y, 1000, BLOCK=1024)
    small = corpus.matmul_dot_kernel.launcher((4, 2), a, b, c, 512, 512, 2048, BM=128, BN=256, BK=64)
    large = corpus.matmul_dot_kernel.launcher((16, 32), big_a, big_b, big_c, 2048, 8192, 256, BM=128, BN=256, BK=64)
    assert small.artifact.plan.notes["split_k"] > 1 and large.artifact.plan.notes["cta_group"] == 2

    def launches():
        softmax()
        small()
        large()

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        launches()                                   # compile, load and warm up outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            launches()
    torch.cuda.synchronize()

    x.copy_(torch.randn(256, 1000, generator=gen, device=device))
    a.copy_((torch.randn(512, 2048, generator=gen, device=device) / 45).bfloat16())
    big_a.copy_((torch.randn(2048, 256, generator=gen, device=device) / 16).bfloat16())
    for out in (y, c, big_c):
        out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    dot_codegen.check_status()
    replayed = [out.clone() for out in (y, c, big_c)]
    for out in (y, c, big_c):
        out.fill_(float("nan"))
    launches()
    torch.cuda.synchronize()
    for got, eager in zip(replayed, (y, c, big_c)):
        assert torch.equal(got, eager)
    assert torch.allclose(y, torch.softmax(x, dim=1), atol=1e-6)
    exact = a.double() @ b.double()
    assert ((c.double() - exact).norm() / exact.norm()).item() < 1e-5


def test_launches_follow_torchs_current_stream(gpu):
    """A kernel launched under `torch.cuda.stream(s)` runs after the work queued on s before it."""
    import torch

    device = torch.device("cuda", 0)
    x = torch.zeros(1 << 22, device=device)
    y = torch.empty_like(x)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(20):
            x.add_(1.0)                              # queued on `stream`; the kernel must see all of it
        corpus.relu_kernel[(x.numel() // 1024,)](x, y, x.numel(), BLOCK=1024)
    stream.synchronize()
    assert float(y.min()) == 20.0 and float(y.max()) == 20.0
