import torch

_COMMS = {}
_NEXT_ID = [1]


def register_communicator(comm):
    cid = _NEXT_ID[0]
    _NEXT_ID[0] += 1
    _COMMS[cid] = comm
    return cid


def set_default_communicator(comm):
    _COMMS[0] = comm
    return 0


def get_communicator(cid=0):
    if cid not in _COMMS:
        raise RuntimeError(f"b200ccl: no communicator registered under id {cid}")
    return _COMMS[cid]


@torch.library.custom_op("b200ccl::all_reduce_out", mutates_args=("out",))
def _all_reduce_out(inp: torch.Tensor, out: torch.Tensor, op: str, comm_id: int) -> None:
    get_communicator(comm_id).all_reduce(out, inp, op=op)


@torch.library.custom_op("b200ccl::all_reduce_inplace", mutates_args=("tensor",))
def _all_reduce_inplace(tensor: torch.Tensor, op: str, comm_id: int) -> None:
    get_communicator(comm_id).all_reduce(tensor, op=op)


@torch.library.custom_op("b200ccl::reduce_scatter_out", mutates_args=("out",))
def _reduce_scatter_out(inp: torch.Tensor, out: torch.Tensor, op: str, comm_id: int) -> None:
    get_communicator(comm_id).reduce_scatter(out, inp, op=op)


@torch.library.custom_op("b200ccl::all_gather_out", mutates_args=("out",))
def _all_gather_out(inp: torch.Tensor, out: torch.Tensor, comm_id: int) -> None:
    get_communicator(comm_id).all_gather(out, inp)


def all_reduce(tensor, op="sum", comm_id=0):
    """Returns the reduction of ``tensor`` over all ranks (out of place)."""
    out = torch.empty_like(tensor)
    torch.ops.b200ccl.all_reduce_out(tensor.contiguous(), out, op, comm_id)
    return out


def all_reduce_(tensor, op="sum", comm_id=0):
    """Reduces ``tensor`` in place over all ranks."""
    torch.ops.b200ccl.all_reduce_inplace(tensor, op, comm_id)
    return tensor


def reduce_scatter(tensor, op="sum", comm_id=0):
    comm = get_communicator(comm_id)
    flat = tensor.contiguous().view(-1)
    out = torch.empty(flat.numel() // comm.world_size, dtype=tensor.dtype, device=tensor.device)
    torch.ops.b200ccl.reduce_scatter_out(flat, out, op, comm_id)
    return out


def all_gather(tensor, comm_id=0):
    comm = get_communicator(comm_id)
    flat = tensor.contiguous().view(-1)
    out = torch.empty(flat.numel() * comm.world_size, dtype=tensor.dtype, device=tensor.device)
    torch.ops.b200ccl.all_gather_out(flat, out, comm_id)
    return out
