"""Concatenation of parameter views that avoids a copy when the views already sit back to
back in one buffer (what `parameters_split` creates). Same role as
miniTransformer/module/_common.py:98-113."""
from typing import Sequence

import torch


class _NoopCat(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dim, *tensors):
        first = tensors[0]
        ctx.dim = dim
        ctx.sizes = [t.shape[dim] for t in tensors]
        if dim != 0 or not _adjacent(tensors):
            return torch.cat(tensors, dim=dim)
        shape = list(first.shape)
        shape[0] = sum(ctx.sizes)
        out = first.new_empty(0)
        out.set_(first.untyped_storage(), first.storage_offset(), shape, first.stride())
        return out

    @staticmethod
    def backward(ctx, grad):
        return (None, *torch.split(grad, ctx.sizes, dim=ctx.dim))


def _adjacent(tensors: Sequence[torch.Tensor]) -> bool:
    first = tensors[0]
    if not first.is_contiguous():
        return False
    ptr = first.data_ptr()
    for t in tensors:
        if (not t.is_contiguous() or t.dtype != first.dtype or t.device != first.device
                or t.shape[1:] != first.shape[1:] or t.data_ptr() != ptr
                or t.untyped_storage().data_ptr() != first.untyped_storage().data_ptr()):
            return False
        ptr += t.numel() * t.element_size()
    return True


def noop_cat(tensors: Sequence[torch.Tensor], dim: int = 0) -> torch.Tensor:
    if not tensors:
        raise ValueError("noop_cat needs at least one tensor")
    if len(tensors) == 1:
        return tensors[0]
    return _NoopCat.apply(dim, *tensors)


_STACKED_OK: dict = {}


def stacked_view(tensors: Sequence[torch.Tensor]):
    """[len(tensors), *shape] view over tensors that sit back to back in one buffer (expert
    weights allocated from one block, or their main_grad buffers), or None when they do not."""
    if not tensors:
        return None
    # the full adjacency walk (contiguity, storage, dtype per tensor) is remembered per set of
    # tensors at these exact addresses: every address is part of the key, so re-pointing any
    # one of them (`.data = ...`, a replaced main_grad) is noticed
    first = tensors[0]
    key = (tuple(t.data_ptr() for t in tensors), tuple(first.shape), tuple(first.stride()), first.dtype,
           first.device)
    ok = _STACKED_OK.get(key)
    if ok is None:
        ok = _adjacent(tensors)
        if len(_STACKED_OK) >= 64:
            _STACKED_OK.clear()
        _STACKED_OK[key] = ok
    if not ok:
        return None
    out = first.detach().new_empty(0)
    out.set_(first.untyped_storage(), first.storage_offset(), [len(tensors), *first.shape],
             [first.numel(), *first.stride()])
    return out
