import torch


def time_cuda(fn, warmup=3, iters=10, stream=None):
    """Mean seconds per call of ``fn`` measured with CUDA events on the launching stream, after
    ``warmup`` untimed calls, with a synchronize on both sides."""
    stream = stream or torch.cuda.current_stream()
    for _ in range(max(warmup, 0)):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(iters):
        fn()
    stop.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / 1e3 / iters
