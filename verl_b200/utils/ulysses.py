"""Function-style API of Ulysses sequence parallelism on [batch, seq, heads, dim]-like tensors: a module-level group,
padding / slicing of the sequence dimension, the sequence <-> head all-to-all (differentiable) and the gather of outputs.
The decoder's hand-scheduled path uses ``models.decoder.UlyssesSequenceParallel``; these functions serve model code written
against autograd.

Parity target: ``verl/utils/ulysses.py`` (group accessors :34-63, ``gather_seq_scatter_heads`` :66,
``gather_heads_scatter_seq`` :90, ``slice_input_tensor`` :121, ``all_to_all_tensor`` :137, ``SeqAllToAll`` :169, ``Gather``
:198, ``gather_outputs_and_unpad`` :247, ``ulysses_pad`` :282, ``ulysses_pad_and_slice_inputs`` :302,
``validate_ulysses_config`` :337).
"""

from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist
from torch import Tensor

__all__ = ["set_ulysses_sequence_parallel_group", "get_ulysses_sequence_parallel_group", "get_ulysses_sequence_parallel_world_size",
           "get_ulysses_sequence_parallel_rank", "gather_seq_scatter_heads", "gather_heads_scatter_seq", "slice_input_tensor",
           "all_to_all_tensor", "all_gather_tensor", "SeqAllToAll", "Gather", "gather_outputs_and_unpad", "ulysses_pad",
           "ulysses_pad_and_slice_inputs", "validate_ulysses_config"]

_GROUP = None


def set_ulysses_sequence_parallel_group(group) -> None:
    global _GROUP
    _GROUP = group


def get_ulysses_sequence_parallel_group():
    return _GROUP


def get_ulysses_sequence_parallel_world_size(group=None) -> int:
    group = group if group is not None else _GROUP
    return dist.get_world_size(group) if group is not None else 1


def get_ulysses_sequence_parallel_rank(group=None) -> int:
    group = group if group is not None else _GROUP
    return dist.get_rank(group) if group is not None else 0


def all_to_all_tensor(local_input: Tensor, scatter_dim: int, gather_dim: int, group=None) -> Tensor:
    """Split ``scatter_dim`` into world-size blocks, exchange, concatenate what arrives along ``gather_dim``."""
    group = group if group is not None else _GROUP
    n = dist.get_world_size(group)
    send = [t.contiguous() for t in torch.tensor_split(local_input, n, dim=scatter_dim)]
    recv = [torch.empty_like(send[0]) for _ in range(n)]
    dist.all_to_all(recv, send, group=group) if local_input.is_cuda else _all_to_all_list(recv, send, group)
    return torch.cat(recv, dim=gather_dim).contiguous()


def _all_to_all_list(recv: list, send: list, group) -> None:
    """List all-to-all through the single-buffer collective (the form every backend implements)."""
    flat_in = torch.stack(send)
    flat_out = torch.empty_like(flat_in)
    dist.all_to_all_single(flat_out, flat_in, group=group)
    for r, o in zip(recv, flat_out):
        r.copy_(o)


def all_gather_tensor(local_tensor: Tensor, group=None, dim: int = 0) -> Tensor:
    group = group if group is not None else _GROUP
    parts = [torch.empty_like(local_tensor) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, local_tensor.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


class SeqAllToAll(torch.autograd.Function):
    """The all-to-all is its own transpose: the backward pass exchanges the other way round."""

    @staticmethod
    def forward(ctx: Any, group, local_input: Tensor, scatter_dim: int, gather_dim: int) -> Tensor:
        ctx.group, ctx.scatter_dim, ctx.gather_dim = group, scatter_dim, gather_dim
        return all_to_all_tensor(local_input, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx: Any, grad_output: Tensor):
        return None, all_to_all_tensor(grad_output, ctx.gather_dim, ctx.scatter_dim, ctx.group), None, None


class Gather(torch.autograd.Function):
    """All-gather along ``gather_dim``; the backward pass keeps this rank's slice of the gradient (scaled by the world
    size when ``grad_scaler``: every rank computed the same loss on the gathered tensor)."""

    @staticmethod
    def forward(ctx: Any, group, local_tensor: Tensor, gather_dim: int, grad_scaler: bool = True) -> Tensor:
        ctx.group, ctx.gather_dim, ctx.grad_scaler = group, gather_dim, grad_scaler
        ctx.world, ctx.rank = dist.get_world_size(group), dist.get_rank(group)
        ctx.part = local_tensor.size(gather_dim)
        return all_gather_tensor(local_tensor, group, dim=gather_dim)

    @staticmethod
    def backward(ctx: Any, grad_output: Tensor):
        if ctx.grad_scaler:
            grad_output = grad_output * ctx.world
        return None, grad_output.split(ctx.part, dim=ctx.gather_dim)[ctx.rank].contiguous(), None, None


def gather_seq_scatter_heads(x: Tensor, seq_dim: int, head_dim: int, unpadded_dim_size: int = 0, group=None) -> Tensor:
    """[.., seq/n, .., heads, ..] -> [.., seq, .., heads/n, ..]; ``unpadded_dim_size`` trims the padding added for slicing."""
    group = group if group is not None else _GROUP
    if group is None:
        return x
    x = SeqAllToAll.apply(group, x, head_dim, seq_dim)
    if unpadded_dim_size and unpadded_dim_size % dist.get_world_size(group) != 0:
        x = x.narrow(seq_dim, 0, unpadded_dim_size)
    return x


def gather_heads_scatter_seq(x: Tensor, head_dim: int, seq_dim: int, group=None) -> Tensor:
    group = group if group is not None else _GROUP
    if group is None:
        return x
    n = dist.get_world_size(group)
    pad = (-x.size(seq_dim)) % n
    if pad:
        x = _pad_tensor(x, seq_dim, pad)
    return SeqAllToAll.apply(group, x, seq_dim, head_dim)


def _pad_tensor(x: Tensor, dim: int, padding_size: int) -> Tensor:
    shape = list(x.shape)
    shape[dim] = padding_size
    return torch.cat([x, torch.zeros(shape, dtype=x.dtype, device=x.device)], dim=dim)


def _unpad_tensor(x: Tensor, dim: int, padding_size: int) -> Tensor:
    return x.narrow(dim, 0, x.size(dim) - padding_size) if padding_size else x


def slice_input_tensor(x: Tensor, dim: int, padding: bool = True, group=None) -> Tensor:
    group = group if group is not None else _GROUP
    n, r = get_ulysses_sequence_parallel_world_size(group), get_ulysses_sequence_parallel_rank(group)
    if n == 1:
        return x
    pad = (-x.size(dim)) % n
    if padding and pad:
        x = _pad_tensor(x, dim, pad)
    part = x.size(dim) // n
    return x.narrow(dim, r * part, part).contiguous()


def gather_outputs_and_unpad(x: Tensor, gather_dim: int, unpad_dim: Optional[int] = None, padding_size: int = 0,
                             grad_scaler: bool = True, group=None) -> Tensor:
    group = group if group is not None else _GROUP
    if group is None:
        return x
    x = Gather.apply(group, x, gather_dim, grad_scaler)
    if unpad_dim is not None and padding_size:
        x = _unpad_tensor(x, unpad_dim, padding_size)
    return x


def ulysses_pad(input_ids_rmpad: Tensor, position_ids_rmpad: Optional[Tensor] = None, sp_size: int = 1):
    """Pad a packed [1, total] stream to a multiple of ``sp_size`` (positions continue counting); returns the pad length."""
    total = input_ids_rmpad.size(1)
    pad = (-total) % sp_size
    if pad:
        input_ids_rmpad = torch.nn.functional.pad(input_ids_rmpad, (0, pad), value=0)
        if position_ids_rmpad is not None:
            extra = torch.arange(pad, device=position_ids_rmpad.device).unsqueeze(0)
            if position_ids_rmpad.dim() == 3:
                extra = extra.unsqueeze(0).expand(position_ids_rmpad.size(0), -1, -1)
            position_ids_rmpad = torch.cat([position_ids_rmpad, extra.to(position_ids_rmpad.dtype)], dim=-1)
    return input_ids_rmpad, position_ids_rmpad, pad


def ulysses_pad_and_slice_inputs(input_ids_rmpad: Tensor, position_ids_rmpad: Optional[Tensor] = None, sp_size: int = 1,
                                 skip_position_ids_rmpad: bool = False):
    input_ids_rmpad, position_ids_rmpad, pad = ulysses_pad(input_ids_rmpad, position_ids_rmpad, sp_size)
    input_ids_rmpad = slice_input_tensor(input_ids_rmpad, dim=1, padding=False)
    if position_ids_rmpad is not None and not skip_position_ids_rmpad:
        position_ids_rmpad = slice_input_tensor(position_ids_rmpad, dim=-1, padding=False)
    return input_ids_rmpad, position_ids_rmpad, pad


def validate_ulysses_config(num_heads: int, ulysses_sequence_size: int) -> None:
    if ulysses_sequence_size > 1:
        assert num_heads % ulysses_sequence_size == 0, \
            f"num_heads ({num_heads}) must be divisible by the sequence-parallel size ({ulysses_sequence_size})"
