"""Shape helpers and collective wrappers (the NCCL / Gloo baseline primitives).

Parity: ``physicsnemo/distributed/utils.py`` — ``compute_split_shapes`` (``:28-44``),
``get_memory_format``, ``pad_helper``, ``truncate_helper``, ``split_tensor_along_dim``
(``:47-110``), ``reduce_loss`` (``:113-150``), ``distributed_transpose`` (``:154-173``), ``_reduce``
/ ``_split`` (``:176-213``), ``all_gather_v_wrapper`` (``:216-296``), ``all_gather_v_bwd_wrapper``
(``:299-372``), ``gather_v_wrapper`` / ``scatter_v_wrapper`` (``:375-538``),
``indexed_all_to_all_v_wrapper`` (+ backward, ``:541-707``), ``mark_module_as_shared`` (``:710-796``).

These are the library-collective statements of each pattern; the peer-memory kernels in
``physicsnemo_b200.parallel.peer`` replace them on the hot paths and are tested against them.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .manager import DistributedManager


def _all_to_all(recv: List[torch.Tensor], send: List[torch.Tensor], group=None, async_op: bool = False):
    """List all-to-all that also works on back ends without a list ``alltoall`` (gloo):
    there the pieces are flattened into one buffer and exchanged with ``all_to_all_single``."""
    backend = dist.get_backend(group)
    if backend == "nccl" or async_op:
        return dist.all_to_all(recv, send, group=group, async_op=async_op)
    in_splits = [t.numel() for t in send]
    out_splits = [t.numel() for t in recv]
    dtype, device = send[0].dtype, send[0].device
    complex_dtype = dtype.is_complex
    flat_in = torch.cat([t.reshape(-1) for t in send]) if sum(in_splits) else torch.empty(0, dtype=dtype, device=device)
    flat_out = torch.empty(sum(out_splits), dtype=dtype, device=device)
    if complex_dtype:
        fi, fo = torch.view_as_real(flat_in).reshape(-1), torch.view_as_real(flat_out).reshape(-1)
        dist.all_to_all_single(fo, fi, [2 * n for n in out_splits], [2 * n for n in in_splits], group=group)
    else:
        dist.all_to_all_single(flat_out, flat_in, out_splits, in_splits, group=group)
    off = 0
    for t, n in zip(recv, out_splits):
        t.copy_(flat_out[off:off + n].reshape(t.shape))
        off += n
    return None


def compute_split_shapes(size: int, num_chunks: int) -> List[int]:
    """Chunk sizes of splitting ``size`` into ``num_chunks``: ceil-div chunks, floor fallback
    when the last chunk would be empty (this rule defines every uneven shard in the package)."""
    if num_chunks == 1:
        return [size]
    chunk = (size + num_chunks - 1) // num_chunks
    last = max(0, size - chunk * (num_chunks - 1))
    if last == 0:
        chunk = size // num_chunks
        last = size - chunk * (num_chunks - 1)
    return [chunk for _ in range(num_chunks - 1)] + [last]


def get_memory_format(tensor: torch.Tensor):
    if tensor.is_contiguous(memory_format=torch.channels_last):
        return torch.channels_last
    return torch.contiguous_format


def pad_helper(tensor: torch.Tensor, dim: int, new_size: int, mode: str = "zero") -> torch.Tensor:
    """Pad ``dim`` to ``new_size`` with zeros or with the conjugate-symmetric continuation."""
    ndim = tensor.ndim
    dim = (dim + ndim) % ndim
    ndim_pad = ndim - dim
    output_shape = [0 for _ in range(2 * ndim_pad)]
    orig_size = tensor.shape[dim]
    output_shape[1] = new_size - orig_size
    tensor_pad = F.pad(tensor, output_shape, mode="constant", value=0.0)
    if mode == "conj":
        lhs = [slice(0, x) if idx != dim else slice(orig_size, new_size) for idx, x in enumerate(tensor.shape)]
        rhs = [slice(0, x) if idx != dim else slice(1, output_shape[1] + 1) for idx, x in enumerate(tensor.shape)]
        tensor_pad[lhs] = torch.flip(torch.conj(tensor_pad[rhs]), dims=[dim])
    return tensor_pad


def truncate_helper(tensor: torch.Tensor, dim: int, new_size: int) -> torch.Tensor:
    ndim = tensor.ndim
    dim = (dim + ndim) % ndim
    sl = [slice(0, x) if idx != dim else slice(0, new_size) for idx, x in enumerate(tensor.shape)]
    return tensor[sl]


def split_tensor_along_dim(tensor: torch.Tensor, dim: int, num_chunks: int):
    if dim >= tensor.dim():
        raise ValueError(f"Error, tensor dimension is {tensor.dim()} which cannot be split along {dim}")
    if tensor.shape[dim] < num_chunks:
        raise ValueError(
            f"Error, cannot split dim {dim} of size {tensor.shape[dim]} into {num_chunks} chunks. "
            "Empty slices are currently not supported."
        )
    return torch.split(tensor, compute_split_shapes(tensor.shape[dim], num_chunks), dim=dim)


@torch.no_grad()
def reduce_loss(loss: float, dst_rank: int = 0, mean: bool = True):
    """Reduce a scalar loss to ``dst_rank`` (mean or sum); other ranks get ``None``."""
    m = DistributedManager()
    t = torch.tensor([loss], device=m.device if dist.is_initialized() and dist.get_backend() == "nccl" else "cpu", dtype=torch.float32)
    if m.distributed and dist.is_initialized() and m.world_size > 1:
        dist.reduce(t, dst_rank, op=dist.ReduceOp.SUM)
        if mean:
            t = t / m.world_size
    return float(t.item()) if m.rank == dst_rank else None


def distributed_transpose(tensor, dim0, dim1, group=None, async_op=False):
    """Pencil transpose: split ``dim0`` into equal chunks, all-to-all, return the received list."""
    input_format = get_memory_format(tensor)
    comm_size = dist.get_world_size(group=group)
    if tensor.shape[dim0] % comm_size:
        raise ValueError(f"dim {dim0} of size {tensor.shape[dim0]} is not divisible by the group size {comm_size}")
    x_send = [y.contiguous(memory_format=input_format) for y in torch.split(tensor, tensor.shape[dim0] // comm_size, dim=dim0)]
    x_recv = [torch.empty_like(x_send[0]) for _ in range(comm_size)]
    req = _all_to_all(x_recv, x_send, group=group, async_op=async_op)
    return x_recv, req


def _reduce(input_, use_fp32=True, group=None):
    """All-reduce (sum); 16-bit floats are summed in fp32."""
    if dist.get_world_size(group=group) == 1:
        return input_
    if use_fp32 and input_.dtype.itemsize < 4 and input_.dtype.is_floating_point:
        dtype = input_.dtype
        inputf = input_.float()
        dist.all_reduce(inputf, group=group)
        return inputf.to(dtype)
    dist.all_reduce(input_, group=group)
    return input_


def _split(input_, dim_, group=None):
    """Keep this rank's chunk of ``dim_`` (chunk sizes from ``compute_split_shapes``)."""
    comm_size = dist.get_world_size(group=group)
    if comm_size == 1:
        return input_
    chunks = split_tensor_along_dim(input_, dim_, comm_size)
    return chunks[dist.get_rank(group=group)].contiguous()


def all_gather_v_wrapper(tensor: torch.Tensor, sizes: Optional[List[int]] = None, dim: int = 0, group=None) -> torch.Tensor:
    """All-gather tensors whose extent along ``dim`` differs per rank; concatenates along ``dim``."""
    comm_size = dist.get_world_size(group=group)
    if sizes is not None and len(sizes) != comm_size:
        raise ValueError("sizes must have one entry per rank")
    if dim >= tensor.dim():
        raise ValueError("dim out of range")
    if comm_size == 1:
        return tensor
    if sizes is None or len(set(sizes)) == 1:
        outs = [torch.empty_like(tensor) for _ in range(comm_size)]
        dist.all_gather(outs, tensor.contiguous(), group=group)
        return torch.cat(outs, dim=dim)
    # uneven: pad every slice to the largest extent (works on every backend), gather, crop
    biggest = max(sizes)
    pad = biggest - tensor.shape[dim]
    if pad:
        pad_shape = list(tensor.shape)
        pad_shape[dim] = pad
        tensor = torch.cat([tensor, tensor.new_zeros(pad_shape)], dim=dim)
    outs = [torch.empty_like(tensor) for _ in range(comm_size)]
    dist.all_gather(outs, tensor.contiguous(), group=group)
    return torch.cat([o.narrow(dim, 0, s) for o, s in zip(outs, sizes)], dim=dim)


def all_gather_v_bwd_wrapper(tensor: torch.Tensor, sizes: List[int], dim: int = 0, use_fp32: bool = True, group=None) -> torch.Tensor:
    """Backward of all-gather-v ("reduce-scatter-v"): every rank receives the sum of its slice."""
    comm_size = dist.get_world_size(group=group)
    rank = dist.get_rank(group=group)
    if len(sizes) != comm_size:
        raise ValueError("sizes must have one entry per rank")
    if comm_size == 1:
        return tensor
    shape = list(tensor.shape)
    shape[dim] = sizes[rank]
    dt = torch.float32 if (use_fp32 and tensor.dtype.itemsize < 4 and tensor.dtype.is_floating_point) else tensor.dtype
    recv = [torch.empty(shape, dtype=dt, device=tensor.device) for _ in range(comm_size)]
    send = [t.to(dt).contiguous() for t in torch.split(tensor, sizes, dim=dim)]
    _all_to_all(recv, send, group=group)
    return torch.stack(recv, dim=0).sum(dim=0).to(tensor.dtype)


def gather_v_wrapper(tensor: torch.Tensor, sizes: List[int], dim: int = 0, dst: int = 0, group=None) -> torch.Tensor:
    """Gather variable-sized slices on ``dst`` (concatenated along ``dim``); others get their input back."""
    comm_size = dist.get_world_size(group=group)
    rank = dist.get_rank(group=group)
    if len(sizes) != comm_size:
        raise ValueError("sizes must have one entry per rank")
    if not 0 <= dst < comm_size:
        raise ValueError("invalid destination rank")
    if tensor.size(dim) != sizes[rank]:
        raise ValueError("local extent does not match sizes[rank]")
    if comm_size == 1:
        return tensor
    shape = list(tensor.shape)
    recv = []
    for r in range(comm_size):
        shape[dim] = sizes[r] if rank == dst else 0
        recv.append(torch.empty(shape, dtype=tensor.dtype, device=tensor.device))
    empty_shape = list(tensor.shape)
    empty_shape[dim] = 0
    send = [tensor.contiguous() if r == dst else torch.empty(empty_shape, dtype=tensor.dtype, device=tensor.device)
            for r in range(comm_size)]
    _all_to_all(recv, send, group=group)
    return torch.cat(recv, dim=dim) if rank == dst else tensor


def scatter_v_wrapper(tensor: torch.Tensor, sizes: List[int], dim: int = 0, src: int = 0, group=None) -> torch.Tensor:
    """Scatter slices of the tensor held by ``src`` (``sizes[r]`` along ``dim`` to rank ``r``)."""
    comm_size = dist.get_world_size(group=group)
    rank = dist.get_rank(group=group)
    if len(sizes) != comm_size:
        raise ValueError("sizes must have one entry per rank")
    if not 0 <= src < comm_size:
        raise ValueError("invalid source rank")
    if comm_size == 1:
        return tensor
    shape = list(tensor.shape)
    recv = []
    for r in range(comm_size):
        shape[dim] = sizes[rank] if r == src else 0
        recv.append(torch.empty(shape, dtype=tensor.dtype, device=tensor.device))
    if rank == src:
        send = [t.contiguous() for t in torch.split(tensor, sizes, dim=dim)]
    else:
        shape[dim] = 0
        send = [torch.empty(shape, dtype=tensor.dtype, device=tensor.device) for _ in range(comm_size)]
    _all_to_all(recv, send, group=group)
    return recv[src]


def indexed_all_to_all_v_wrapper(tensor: torch.Tensor, indices: List[torch.Tensor], sizes: List[List[int]],
                                 dim: int = 0, group=None) -> torch.Tensor:
    """Send ``tensor[indices[r]]`` (along ``dim``) to every rank ``r``; concatenate what arrives.

    ``sizes[i][j]`` is the number of rows rank ``i`` sends to rank ``j``.
    """
    comm_size = dist.get_world_size(group=group)
    rank = dist.get_rank(group=group)
    if len(sizes) != comm_size or len(sizes[0]) != comm_size or len(indices) != comm_size:
        raise ValueError("sizes / indices must have one entry per rank")
    x_send = [tensor.index_select(dim, idx.to(torch.long)) if dim != 0 else tensor[idx] for idx in indices]
    if comm_size == 1:
        return x_send[0]
    shape = list(tensor.shape)
    x_recv = []
    for r in range(comm_size):
        shape[dim] = sizes[r][rank]
        x_recv.append(torch.empty(shape, dtype=tensor.dtype, device=tensor.device))
    _all_to_all(x_recv, [x.contiguous() for x in x_send], group=group)
    return torch.cat(x_recv, dim=dim)


def indexed_all_to_all_v_wrapper_bwd(tensor: torch.Tensor, indices: List[torch.Tensor], sizes: List[List[int]],
                                     tensor_size_along_dim: int, use_fp32: bool = True, dim: int = 0,
                                     group=None) -> torch.Tensor:
    """Backward of ``indexed_all_to_all_v``: return the pieces to their senders and ``index_add``."""
    comm_size = dist.get_world_size(group=group)
    rank = dist.get_rank(group=group)
    if len(sizes) != comm_size or len(sizes[0]) != comm_size or len(indices) != comm_size:
        raise ValueError("sizes / indices must have one entry per rank")
    shape = list(tensor.shape)
    recv_sizes = [sizes[i][rank] for i in range(comm_size)]
    send_sizes = [sizes[rank][i] for i in range(comm_size)]
    x_send = [t.contiguous() for t in torch.split(tensor, recv_sizes, dim=dim)]
    x_recv = []
    for r in range(comm_size):
        shape[dim] = send_sizes[r]
        x_recv.append(torch.empty(shape, dtype=tensor.dtype, device=tensor.device))
    if comm_size > 1:
        _all_to_all(x_recv, x_send, group=group)
    else:
        x_recv = x_send
    idx = torch.cat(indices, dim=0).to(torch.long)
    x_cat = torch.cat(x_recv, dim=dim)
    shape[dim] = tensor_size_along_dim
    dt = torch.float32 if (use_fp32 and tensor.dtype.itemsize < 4 and tensor.dtype.is_floating_point) else tensor.dtype
    out = torch.zeros(shape, dtype=dt, device=tensor.device)
    out.index_add_(dim, idx, x_cat.to(dt))
    return out.to(tensor.dtype)


def mark_module_as_shared(module: torch.nn.Module, process_group: Optional[str], recurse: bool = True,
                          use_fp32_reduction: bool = True) -> torch.nn.Module:
    """Mark parameters as shared over a named group: their gradients are all-reduced after
    accumulation (post-accumulate-grad hook)."""
    group = DistributedManager().group(process_group)
    handle_key = "_shared_weight_dist_hook"

    def hook(param: torch.Tensor) -> None:
        param.grad = _reduce(param.grad, group=group, use_fp32=use_fp32_reduction)

    def already_marked_hook(mod, _inputs):
        raise RuntimeError(f"Module {mod} is already marked as shared in {process_group}.")

    for name, param in module.named_parameters(recurse=recurse):
        if hasattr(param, handle_key):
            raise RuntimeError(f"Parameter {name} already marked as having shared weights, can't mark it again!")
        setattr(param, handle_key, param.register_post_accumulate_grad_hook(hook))
    return module


def unmark_module_as_shared(module: torch.nn.Module, recurse: bool = True) -> torch.nn.Module:
    handle_key = "_shared_weight_dist_hook"
    for name, param in module.named_parameters(recurse=recurse):
        if not hasattr(param, handle_key):
            raise RuntimeError(f"Parameter {name} NOT marked as having shared weights, can't unmark it!")
        getattr(param, handle_key).remove()
        delattr(param, handle_key)
    return module
