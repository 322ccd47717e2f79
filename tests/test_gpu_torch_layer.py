"""PyTorch layer on one GPU: custom ops, CUDA-graph capture and replay of a collective, the
bucketed reducer and the data-parallel wrapper over a one-rank communicator (the kernels and the
launch path are the real ones; with one rank the reduction is the identity / a scale by 1)."""
import pytest
import torch

import nano_nccl_b200 as nn
from nano_nccl_b200 import ops
from nano_nccl_b200.models import TinyGPT2
from nano_nccl_b200.parallel import BucketAllReducer, CclBackend, DistributedDataParallel

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm():
    torch.cuda.set_device(0)
    c = nn.Communicator(devices=[0], wait_timeout_ms=2000)
    yield c
    c.close()


def test_custom_ops(comm):
    cid = ops.register_communicator(comm)
    x = torch.randn(4096, device="cuda", dtype=torch.bfloat16)
    y = ops.all_reduce(x, "sum", cid)
    assert torch.equal(y, x)
    z = x.clone()
    torch.ops.b200ccl.all_reduce_inplace(z, "avg", cid)
    torch.cuda.synchronize()
    assert torch.equal(z, x)
    assert torch.equal(ops.all_gather(x, cid), x) and torch.equal(ops.reduce_scatter(x, "sum", cid), x)
    comm.check_async_error()


def test_cuda_graph_capture_and_replay(comm):
    x = comm.empty(1 << 16, torch.float32)
    y = comm.empty(1 << 16, torch.float32)
    x.normal_()
    comm.all_reduce(y, x)  # eager call first: the capture below must not depend on its event
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(3):
            comm.all_reduce(y, x, op="sum")
    for round_ in range(3):
        x.fill_(float(round_ + 1))
        y.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, x)
    comm.all_reduce(y, x)  # eager again after the capture
    torch.cuda.synchronize()
    comm.check_async_error()


def test_bucket_reducer_and_ddp_on_symmetric_buckets(comm):
    backend = CclBackend(comm)
    tensors = [torch.randn(n, device="cuda", dtype=torch.bfloat16) for n in (5, 70000, 33, 200000)]
    want = [t.clone() for t in tensors]
    red = BucketAllReducer(backend, [t.numel() for t in tensors], torch.bfloat16, "cuda:0", bucket_bytes=256 << 10, op="avg")
    assert red.plan.num_buckets >= 2
    red.reduce(tensors)
    torch.cuda.synchronize()
    for a, b in zip(tensors, want):
        assert torch.equal(a, b)
    model = TinyGPT2(vocab=64, context=16, hidden=32, layers=1, heads=2).cuda()
    ref = TinyGPT2(vocab=64, context=16, hidden=32, layers=1, heads=2).cuda()
    ref.load_state_dict(model.state_dict())
    ddp = DistributedDataParallel(model, backend, bucket_bytes=64 << 10)
    tokens = torch.randint(0, 64, (2, 16), device="cuda")
    ddp(tokens).float().logsumexp(-1).mean().backward()
    ddp.finish()
    ref(tokens).float().logsumexp(-1).mean().backward()
    torch.cuda.synchronize()
    comm.check_async_error()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-5)
