"""A small data-parallel wrapper: gradients are views into symmetric buckets, each bucket is
all-reduced (avg) on a side stream as soon as all of its gradients have been produced, and
``finish()`` orders the optimizer's stream behind the reductions."""
import torch

from .bucket import BucketAllReducer


class DistributedDataParallel(torch.nn.Module):
    def __init__(self, module, backend, bucket_bytes=25 << 20):
        super().__init__()
        self.module = module
        params = [p for p in module.parameters() if p.requires_grad]
        # Gradients become ready roughly in reverse registration order: bucket them that way.
        self.params = list(reversed(params))
        if not self.params:
            raise ValueError("module has no trainable parameters")
        dtype, device = self.params[0].dtype, self.params[0].device
        if any(p.dtype != dtype or p.device != device for p in self.params):
            raise ValueError("all parameters must share one dtype and device")
        self.reducer = BucketAllReducer(backend, [p.numel() for p in self.params], dtype, device, bucket_bytes, op="avg")
        views = self.reducer.views([p.shape for p in self.params])
        self._pending = [0] * self.reducer.plan.num_buckets
        self._bucket_of = {}
        for p, v, (b, _, _) in zip(self.params, views, self.reducer.plan.slots):
            p.grad = v  # gradients accumulate straight into the bucket
            self._bucket_of[p] = b
            p.register_post_accumulate_grad_hook(self._on_grad)
        self._reset()

    def _reset(self):
        for b in range(len(self._pending)):
            self._pending[b] = len(self.reducer.plan.tensors_of(b))

    def _on_grad(self, p):
        b = self._bucket_of[p]
        self._pending[b] -= 1
        if self._pending[b] == 0:
            self.reducer.reduce_bucket(b)

    def forward(self, *args, **kw):
        return self.module(*args, **kw)

    def finish(self):
        """Call after backward(): waits (on the stream) for all buckets and re-arms the hooks."""
        for b, left in enumerate(self._pending):
            if left > 0:  # parameters that received no gradient this step
                self.reducer.reduce_bucket(b)
        self.reducer.wait()
        self._reset()

    def zero_grad(self, set_to_none=False):
        for b in self.reducer.buckets:
            b.zero_()
