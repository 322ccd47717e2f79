"""Python face of the communicator: create one per process (one GPU each) or one for several
GPUs of this process, and run all_reduce / reduce_scatter / all_gather on torch tensors.

The reference library (nano-nccl) has no Python layer; its C++ calls
(include/nano_nccl/communicator.h:31-58) are what these methods forward to.
"""
import ctypes
import os

import torch

from . import _lib

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_OPS = {"sum": 0, "avg": 1, "max": 2, "min": 3}
_COLL = {"all_reduce": 0, "reduce_scatter": 1, "all_gather": 2}
_ALGO_NAMES = ["auto", "oneshot", "twoshot", "nvls", "ring", "ll", "copy", "pipeline"]


class _SymmetricBlock:
    """Owner of one symmetric allocation; exposes it to torch through the CUDA array interface."""

    def __init__(self, comm, ptr, nbytes):
        self.comm, self.ptr, self.nbytes = comm, ptr, nbytes
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


class Communicator:
    """One communicator.

    * ``Communicator(devices=[0, 1, ...])`` — this process drives all listed GPUs (tensors are then
      passed as lists, one per GPU).
    * ``Communicator.from_env()`` / ``Communicator(rank=, world_size=, addr=, port=)`` — one process
      per GPU; peer memory is shared through exported allocations.
    * ``Communicator(devices=[0], loopback_ranks=N)`` — N ranks emulated on one GPU (tests, profiling).
    """

    def __init__(self, devices=None, rank=None, world_size=None, addr="127.0.0.1", port=None,
                 transport="auto", algo="auto", loopback_ranks=0, wait_timeout_ms=0.0,
                 staging_bytes=0, enable_nvls=True, channels=0, max_ctas=0):
        lib = _lib.load()
        self._lib = lib
        self._handle = ctypes.c_void_p()
        self._bootstrap = ctypes.c_void_p()
        self._blocks = []
        cfg = _lib.B2Config()
        lib.b2_config_default(ctypes.byref(cfg))
        t, a = ctypes.c_int(), ctypes.c_int()
        if lib.b2_parse_transport(transport.encode(), ctypes.byref(t)) != 0 and transport != "socket":
            raise ValueError(f"unknown transport '{transport}'")
        cfg.transport = 3 if transport == "socket" else t.value
        if lib.b2_parse_algo(algo.encode(), ctypes.byref(a)) != 0:
            raise ValueError(f"unknown algo '{algo}'")
        cfg.algo = a.value
        cfg.loopback = 1 if loopback_ranks else 0
        cfg.loopback_ranks = int(loopback_ranks)
        cfg.wait_timeout_ms = float(wait_timeout_ms)
        cfg.staging_bytes = int(staging_bytes)
        cfg.enable_nvls = 1 if enable_nvls else 0
        cfg.channels = int(channels)
        cfg.max_ctas = int(max_ctas)
        if devices is None:
            devices = [torch.cuda.current_device()]
        self.devices = list(devices)
        dev_arr = (ctypes.c_int * len(self.devices))(*self.devices)
        if world_size is not None and world_size > 1:
            if port is None:
                raise ValueError("multi-process communicator needs a port")
            _lib.check(lib.b2_bootstrap_create(addr.encode(), int(port), int(rank), int(world_size), 120000,
                                               ctypes.byref(self._bootstrap)))
            _lib.check(lib.b2_comm_create_bootstrap(self._bootstrap, dev_arr, len(self.devices), ctypes.byref(cfg),
                                                    ctypes.byref(self._handle)))
        else:
            _lib.check(lib.b2_comm_create(dev_arr, len(self.devices), ctypes.byref(cfg), ctypes.byref(self._handle)))
        self.local_ranks = lib.b2_comm_local_ranks(self._handle)
        self.world_size = lib.b2_comm_global_ranks(self._handle)
        self.rank = lib.b2_comm_first_rank(self._handle)
        self._one = ((ctypes.c_void_p * 1)(), (ctypes.c_void_p * 1)(), (ctypes.c_void_p * 1)())

    @classmethod
    def from_env(cls, port=None, **kw):
        """One process per GPU, laid out by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR (torchrun).

        The rendezvous port defaults to B200CCL_PORT, else MASTER_PORT + 1000 + 7."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        local = int(os.environ.get("LOCAL_RANK", str(rank)))
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        if port is None:
            port = int(os.environ.get("B200CCL_PORT", int(os.environ.get("MASTER_PORT", "29500")) + 1007))
        torch.cuda.set_device(local)
        return cls(devices=[local], rank=rank, world_size=world, addr=addr, port=port, **kw)

    # -- properties -------------------------------------------------------------------------
    @property
    def transport(self):
        return self._lib.b2_transport_name(self._lib.b2_comm_transport(self._handle)).decode()

    @property
    def nvls(self):
        return bool(self._lib.b2_comm_nvls(self._handle))

    def describe(self):
        n = self._lib.b2_comm_describe(self._handle, None, 0)
        buf = ctypes.create_string_buffer(n + 1)
        self._lib.b2_comm_describe(self._handle, buf, n + 1)
        return buf.value.decode()

    def last_call(self):
        out = (ctypes.c_int * 7)()
        self._lib.b2_comm_last_call(self._handle, out)
        return {"algo": _ALGO_NAMES[out[0]], "grid": out[1], "block": out[2], "staged_in": bool(out[3]),
                "staged_out": bool(out[4]), "vectorized": bool(out[5]), "pack_bytes": out[6]}

    def ring_channel(self, local_rank=0, channel=0):
        """Addresses one local rank's ring channel is wired to (after a ring collective has run)."""
        out = (ctypes.c_void_p * 8)()
        _lib.check(self._lib.b2_comm_ring_channel(self._handle, int(local_rank), int(channel), out))
        names = ("send_fifo", "recv_fifo", "send_tail", "send_head", "recv_tail", "recv_head", "send_base", "recv_base")
        return {k: int(v or 0) for k, v in zip(names, out)}

    def check_async_error(self):
        _lib.check(self._lib.b2_comm_check_async_error(self._handle))

    # -- symmetric memory ----------------------------------------------------------------------
    def empty(self, shape, dtype=torch.float32):
        """Symmetric tensor(s): mapped on every peer (and multicast-bound when NVLS is available), so
        collectives on them need no staging. COLLECTIVE: every process calls it with the same shape, in
        the same order. Returns one tensor (one local rank) or a list (several local GPUs)."""
        if isinstance(shape, int):
            shape = (shape,)
        numel = 1
        for s in shape:
            numel *= int(s)
        esize = torch.empty((), dtype=dtype).element_size()
        nbytes = max(numel * esize, 16)
        ptrs = (ctypes.c_void_p * self.local_ranks)()
        _lib.check(self._lib.b2_comm_alloc_symmetric(self._handle, nbytes, ptrs))
        outs = []
        for i in range(self.local_ranks):
            dev = self.devices[0] if len(self.devices) == 1 else self.devices[i]
            block = _SymmetricBlock(self, ptrs[i], nbytes)
            self._blocks.append(block)
            with torch.cuda.device(dev):
                raw = torch.as_tensor(block, device=f"cuda:{dev}")
            outs.append(raw[: numel * esize].view(dtype).view(*shape))
        return outs[0] if self.local_ranks == 1 else outs

    def register(self, tensors):
        """Registers ordinary CUDA tensor(s) (one per local rank) so that peers address them directly:
        later collectives on them, or on slices at the same offset on every rank, skip the staging copy.
        COLLECTIVE: every process calls it with a tensor of the same size, in the same order. Keep the
        tensors alive until ``unregister``. Tensors from the virtual-memory (expandable segments)
        allocator cannot be shared this way; use ``empty()`` for those."""
        if isinstance(tensors, torch.Tensor):
            tensors = [tensors]
        if len(tensors) != self.local_ranks:
            raise ValueError(f"need one tensor per local rank ({self.local_ranks})")
        ptrs = (ctypes.c_void_p * self.local_ranks)(*[t.data_ptr() for t in tensors])
        _lib.check(self._lib.b2_comm_register(self._handle, ptrs, tensors[0].numel() * tensors[0].element_size()))

    def unregister(self, tensors):
        if isinstance(tensors, torch.Tensor):
            tensors = [tensors]
        ptrs = (ctypes.c_void_p * self.local_ranks)(*[t.data_ptr() for t in tensors])
        _lib.check(self._lib.b2_comm_unregister(self._handle, ptrs))

    # -- collectives -----------------------------------------------------------------------------
    def _device_index(self, i):
        return self.devices[0] if len(self.devices) == 1 else self.devices[i]

    def _check_tensor(self, what, i, t, dtype, numel):
        """Everything the C layer cannot see behind a raw pointer: a tensor that is too small, of
        another dtype or on another GPU would make the kernel write outside the allocation."""
        if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{what}[{i}] must be a contiguous CUDA tensor")
        if t.dtype != dtype:
            raise ValueError(f"{what}[{i}] has dtype {t.dtype}, expected {dtype}")
        if t.numel() != numel:
            raise ValueError(f"{what}[{i}] has {t.numel()} elements, expected {numel}")
        want = self._device_index(i)
        if t.device.index != want:
            raise ValueError(f"{what}[{i}] lives on cuda:{t.device.index}, local rank {i} of this communicator drives cuda:{want}")

    def _run(self, coll, outs, inps, op, streams, count, in_numel, out_numel, in_place=False):
        if op not in _OPS:
            raise ValueError(f"unknown reduction '{op}'")
        if isinstance(inps, torch.Tensor):
            # Fast path: one local rank, one tensor each way.
            if self.local_ranks != 1 or not isinstance(outs, torch.Tensor):
                raise ValueError(f"need one tensor per local rank ({self.local_ranks})")
            dtype = inps.dtype
            code = _DTYPES.get(dtype)
            if code is None:
                raise ValueError(f"unsupported dtype {dtype}")
            self._check_tensor("input", 0, inps, dtype, in_numel)
            self._check_tensor("output", 0, outs, dtype, out_numel)
            if streams is None:
                sp = torch.cuda.current_stream(inps.device).cuda_stream
            else:
                s0 = streams[0] if isinstance(streams, (list, tuple)) else streams
                sp = s0.cuda_stream if hasattr(s0, "cuda_stream") else int(s0)
            a = self._one
            a[0][0], a[1][0], a[2][0] = inps.data_ptr(), outs.data_ptr(), sp
            rc = self._lib.b2_collective(self._handle, _COLL[coll], a[0], a[1], a[2], count, code, _OPS[op], 1 if in_place else 0)
            if rc != 0:
                _lib.check(rc)
            return
        if isinstance(outs, torch.Tensor) or len(inps) != self.local_ranks or len(outs) != self.local_ranks:
            raise ValueError(f"need one tensor per local rank ({self.local_ranks})")
        dtype = inps[0].dtype
        if dtype not in _DTYPES:
            raise ValueError(f"unsupported dtype {dtype}")
        for i, (x, y) in enumerate(zip(inps, outs)):
            self._check_tensor("input", i, x, dtype, in_numel)
            self._check_tensor("output", i, y, dtype, out_numel)
        if streams is None:
            streams = [torch.cuda.current_stream(t.device).cuda_stream for t in inps]
        elif not isinstance(streams, (list, tuple)):
            streams = [streams] * len(inps)
        if len(streams) != self.local_ranks:
            raise ValueError(f"need one stream per local rank ({self.local_ranks})")
        streams = [s.cuda_stream if hasattr(s, "cuda_stream") else int(s) for s in streams]
        n = self.local_ranks
        send = (ctypes.c_void_p * n)(*[t.data_ptr() for t in inps])
        recv = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outs])
        st = (ctypes.c_void_p * n)(*streams)
        _lib.check(self._lib.b2_collective(self._handle, _COLL[coll], send, recv, st, count, _DTYPES[dtype], _OPS[op],
                                           1 if in_place else 0))

    def all_reduce(self, out, inp=None, op="sum", stream=None):
        """out = reduce(inp over all ranks). ``inp=None`` (or the same tensor) reduces in place."""
        if inp is None:
            inp = out
        first_in = inp if isinstance(inp, torch.Tensor) else inp[0]
        first_out = out if isinstance(out, torch.Tensor) else out[0]
        in_place = first_in.data_ptr() == first_out.data_ptr()
        n = first_in.numel()
        self._run("all_reduce", out, inp, op, stream, n, n, n, in_place)
        return out

    def reduce_scatter(self, out, inp, op="sum", stream=None):
        """Rank r's ``out`` (numel = inp.numel() / world_size) receives block r of the reduction."""
        first_out = out if isinstance(out, torch.Tensor) else out[0]
        first_in = inp if isinstance(inp, torch.Tensor) else inp[0]
        if first_in.numel() != first_out.numel() * self.world_size:
            raise ValueError("reduce_scatter: input must hold world_size blocks of the output's size")
        n = first_out.numel()
        self._run("reduce_scatter", out, inp, op, stream, n, n * self.world_size, n)
        return out

    def all_gather(self, out, inp, stream=None):
        """``out`` (numel = inp.numel() * world_size) receives every rank's ``inp``, in rank order."""
        first_out = out if isinstance(out, torch.Tensor) else out[0]
        first_in = inp if isinstance(inp, torch.Tensor) else inp[0]
        if first_out.numel() != first_in.numel() * self.world_size:
            raise ValueError("all_gather: output must hold world_size blocks of the input's size")
        n = first_in.numel()
        self._run("all_gather", out, inp, "sum", stream, n, n, n * self.world_size)
        return out

    def free(self, tensors):
        """Releases the symmetric allocation behind tensor(s) returned by ``empty()``. COLLECTIVE: every
        process calls it for the same allocation, in the same order. The tensors (and every view of
        them) must not be used afterwards: their memory is unmapped."""
        if isinstance(tensors, torch.Tensor):
            tensors = [tensors]
        if len(tensors) != self.local_ranks:
            raise ValueError(f"need one tensor per local rank ({self.local_ranks})")
        ptrs = (ctypes.c_void_p * self.local_ranks)(*[t.data_ptr() for t in tensors])
        _lib.check(self._lib.b2_comm_free_symmetric(self._handle, ptrs))
        gone = {int(p) for p in ptrs}
        self._blocks = [b for b in self._blocks if int(b.ptr) not in gone]

    def close(self):
        if self._handle:
            self._lib.b2_comm_destroy(self._handle)
            self._handle = ctypes.c_void_p()
        if self._bootstrap:
            self._lib.b2_bootstrap_destroy(self._bootstrap)
            self._bootstrap = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.close()
        return False

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
