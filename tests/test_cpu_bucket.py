"""Host-side logic of the PyTorch layer on CPU: bucket planning, and the bucketed reducer and the
data-parallel wrapper over torch.distributed with the gloo backend (two real processes)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from nano_nccl_b200.models import gpt2_small_shapes
from nano_nccl_b200.parallel import BucketPlan

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bucket_plan_packs_in_order_and_aligns():
    plan = BucketPlan([10, 20, 5, 40, 3], element_size=2, bucket_bytes=64, align=8)  # 32 elements per bucket
    # 10 pads to 16; 16 + 20 would exceed 32 → second bucket; 20 pads to 24, 5 fits behind it.
    assert [s[0] for s in plan.slots] == [0, 1, 1, 2, 3]
    # offsets are 16-byte aligned inside a bucket (8 two-byte elements)
    assert plan.slots[2][1] == 24 and all(off % 8 == 0 for _, off, _ in plan.slots)
    assert all(n % 8 == 0 for n in plan.bucket_numel)
    assert plan.tensors_of(1) == [1, 2] and plan.num_buckets == 4
    # a tensor larger than the bucket size gets a bucket of its own
    assert plan.bucket_numel[2] == 40


def test_gpt2_small_stack_is_124m_elements_in_25mib_buckets():
    shapes = gpt2_small_shapes()
    numels = [int(torch.Size(s).numel()) for s in shapes]
    total = sum(numels)
    assert 124_000_000 < total < 125_000_000
    plan = BucketPlan(numels, element_size=2, bucket_bytes=25 << 20)
    cap = (25 << 20) // 2
    for b, n in enumerate(plan.bucket_numel):
        assert n <= cap or len(plan.tensors_of(b)) == 1  # only a single oversize tensor may exceed the cap
    assert sum(plan.bucket_numel) >= total
    with pytest.raises(ValueError):
        BucketPlan([1], 2, bucket_bytes=0)


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["B2_ROOT"])
from nano_nccl_b200.parallel import BucketAllReducer, DistributedDataParallel, TorchDistBackend
from nano_nccl_b200.models import TinyGPT2
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, world = dist.get_rank(), dist.get_world_size()
backend = TorchDistBackend()
torch.manual_seed(100 + rank)
tensors = [torch.randn(n) for n in (5, 1000, 37, 4096, 1)]
expect = [t.clone() for t in tensors]
for t in expect:
    dist.all_reduce(t); t.div_(world)
red = BucketAllReducer(backend, [t.numel() for t in tensors], torch.float32, "cpu", bucket_bytes=4096 * 4, op="avg")
assert red.plan.num_buckets >= 2
red.reduce(tensors)
for a, b in zip(tensors, expect):
    assert torch.allclose(a, b, atol=1e-6)
assert red.launches == red.plan.num_buckets
# data-parallel wrapper: gradients live in the buckets and end up averaged over ranks
torch.manual_seed(0)
model = TinyGPT2(vocab=64, context=16, hidden=32, layers=1, heads=2)
ddp = DistributedDataParallel(model, backend, bucket_bytes=64 * 1024)
torch.manual_seed(200 + rank)
tokens = torch.randint(0, 64, (2, 16))
loss = ddp(tokens).float().logsumexp(-1).mean()
loss.backward()
ddp.finish()
grads = [p.grad.clone() for p in ddp.params]
# reference: the same loss on every rank's data, averaged
ref_model = TinyGPT2(vocab=64, context=16, hidden=32, layers=1, heads=2)
ref_model.load_state_dict(model.state_dict())
ref_loss = ref_model(tokens).float().logsumexp(-1).mean()
ref_loss.backward()
for p, g in zip(reversed([q for q in ref_model.parameters()]), grads):
    r = p.grad.clone(); dist.all_reduce(r); r.div_(world)
    assert torch.allclose(g, r, atol=1e-5), (g - r).abs().max()
dist.barrier()
print("BUCKET WORKER OK")
"""


def test_bucket_reducer_and_ddp_over_gloo(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), B2_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate(timeout=180)
        assert p.returncode == 0 and "BUCKET WORKER OK" in out, out
