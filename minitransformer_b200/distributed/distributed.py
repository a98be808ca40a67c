"""Tensor-parallel collectives used by the linear modules: thin wrappers over
torch.distributed on the caller's process group (NCCL over NVLink on GPUs, gloo in the CPU
tests). Same entry points as miniTransformer/distributed/distributed.py:13-121, plus the
packed quantized all-gather this implementation adds."""
import os
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..utils.utils import FP8_DTYPES

_TP_ATTRS = {"tensor_model_parallel": False, "partition_dim": -1, "partition_stride": 1}


def get_distributed_world_size(group=None) -> int:
    return dist.get_world_size(group=group) if dist.is_initialized() else 1


def get_distributed_rank(group=None) -> int:
    return dist.get_rank(group=group) if dist.is_initialized() else 0


def set_tensor_model_parallel_attributes(tensor: torch.Tensor, is_parallel: bool, dim: int, stride: int) -> None:
    for name in _TP_ATTRS:
        assert not hasattr(tensor, name), f"{name} already set"
    tensor.tensor_model_parallel = is_parallel
    tensor.partition_dim = dim
    tensor.partition_stride = stride


def reduce_scatter_along_first_dim(input: torch.Tensor, tp_group, async_op: bool = False):
    world = get_distributed_world_size(tp_group)
    if world == 1:
        return input, None
    assert input.shape[0] % world == 0, "first dimension must divide by the tensor-parallel size"
    out = torch.empty((input.shape[0] // world, *input.shape[1:]), dtype=input.dtype, device=input.device)
    handle = dist.reduce_scatter_tensor(out, input.contiguous(), group=tp_group, async_op=async_op)
    return out, handle


def gather_along_first_dim(input: torch.Tensor, process_group, async_op: bool = False):
    world = get_distributed_world_size(process_group)
    if world == 1:
        return input, None
    out = torch.empty((input.shape[0] * world, *input.shape[1:]), dtype=input.dtype, device=input.device)
    src, dst = input.contiguous(), out
    if input.dtype in FP8_DTYPES:  # byte view: collectives need not know the 8-bit float types
        src, dst = src.view(torch.uint8), dst.view(torch.uint8)
    handle = dist.all_gather_into_tensor(dst, src, group=process_group, async_op=async_op)
    return out, handle


def allreduce(input_: torch.Tensor, tp_group=None, async_op: bool = False):
    if get_distributed_world_size(tp_group) == 1:
        return input_, None
    handle = dist.all_reduce(input_, group=tp_group, async_op=async_op)
    return input_, handle


def allreduce_max_(scalars: torch.Tensor, tp_group) -> torch.Tensor:
    """In-place MAX all-reduce of a few fp32 scalars (the per-tensor abs-max values), so that
    every rank quantizes its shard with the scale of the gathered tensor."""
    if get_distributed_world_size(tp_group) > 1:
        dist.all_reduce(scalars, op=dist.ReduceOp.MAX, group=tp_group)
    return scalars


def gather_packed_along_first_dim(parts: Sequence[torch.Tensor], process_group) -> Tuple[torch.Tensor, ...]:
    """All-gathers several byte tensors that share their first-dim sharding with ONE collective:
    each rank packs [codes | scales | ...] of its shard into one buffer; after the gather the
    pieces are re-assembled per tensor in rank order along dim 0."""
    world = get_distributed_world_size(process_group)
    if world == 1:
        return tuple(parts)
    flat = [p.contiguous().view(torch.uint8).reshape(-1) for p in parts]
    sizes = [f.numel() for f in flat]
    packed = torch.cat(flat)
    out = torch.empty(world * packed.numel(), dtype=torch.uint8, device=packed.device)
    dist.all_gather_into_tensor(out, packed, group=process_group)
    out = out.view(world, packed.numel())
    res, off = [], 0
    for p, n in zip(parts, sizes):
        piece = out[:, off:off + n].contiguous().reshape(-1)          # bytes of all ranks, rank-major
        if p.dtype != torch.uint8:
            piece = piece.view(p.dtype)
        res.append(piece.reshape(world * p.shape[0], *p.shape[1:]))
        off += n
    return tuple(res)


def _coalesce_gathers(world: int) -> bool:
    """One coalesced launch or one collective per tensor: MT_TP_COALESCE=0/1 decides, else the
    measured preference (separate collectives on 2 ranks, where the coalesced form was slower)."""
    v = os.environ.get("MT_TP_COALESCE")
    if v is not None:
        return v not in ("0", "")
    return world >= 4


def _gather_many_bytes(tensors, out_shapes, process_group, async_op: bool = False):
    """All-gathers several contiguous tensors as bytes, each rank-major into a new tensor of the
    given shape, as ONE coalesced NCCL launch where the backend offers it (the per-collective
    latency is what counts for the small scale tensors, above all on 8 ranks); otherwise one
    collective per tensor. Returns (outputs, handles)."""
    world = get_distributed_world_size(process_group)
    srcs = [t.contiguous().view(torch.uint8).reshape(-1) for t in tensors]
    outs = [torch.empty(world * s.numel(), dtype=torch.uint8, device=s.device) for s in srcs]
    group = process_group if process_group is not None else dist.group.WORLD
    handles = []
    coalesced = getattr(group, "allgather_into_tensor_coalesced", None)
    done = False
    if coalesced is not None and len(srcs) > 1 and srcs[0].is_cuda and _coalesce_gathers(world):
        try:
            work = coalesced(outs, srcs)
            if async_op:
                handles.append(work)
            else:
                work.wait()
            done = True
        except (RuntimeError, NotImplementedError, TypeError):
            done = False
    if not done:
        for o, s_ in zip(outs, srcs):
            handles.append(dist.all_gather_into_tensor(o, s_, group=process_group, async_op=async_op))
    return [o.view(*shape) for o, shape in zip(outs, out_shapes)], [h for h in handles if h is not None]


def gather_gemm_ready(data: torch.Tensor, scale_swz: torch.Tensor, process_group, data_t=None, scale_t_swz=None,
                      async_op: bool = False):
    """Gathers a token-sharded quantized tensor in the form the GEMMs read, with no copy after
    the collective.
    * Row-wise codes [rows, bytes] are concatenated along rows; GEMM-layout scales are gathered
      as they are: with shards of whole 128-row chunks the ranks' chunk lists follow one another.
    * The transposed copy of rank r, [features, tokens / world], is slab r of the contraction
      dimension of the gathered x^T; the result [world, features, bytes] (and the per-rank
      GEMM-layout scale buffers back to back) is what the K-slab GEMM entry points take.
    Returns (codes, scales, codes_t or None, scales_t or None, handles)."""
    world = get_distributed_world_size(process_group)
    assert data.shape[0] % 128 == 0, "row shards must be multiples of 128 rows"
    tensors = [data, scale_swz]
    shapes = [(world * data.shape[0], data.shape[1] * data.element_size()), (world * scale_swz.numel(),)]
    if data_t is not None:
        tensors += [data_t, scale_t_swz]
        shapes += [(world, data_t.shape[0], data_t.shape[1] * data_t.element_size()), (world * scale_t_swz.numel(),)]
    outs, handles = _gather_many_bytes(tensors, shapes, process_group, async_op)
    if data_t is None:
        outs += [None, None]
    return outs[0], outs[1], outs[2], outs[3], handles


def gather_transposed_as_k_slabs(data_t: torch.Tensor, scale_t_swz: torch.Tensor, process_group,
                                 async_op: bool = False):
    """The transposed half of gather_gemm_ready on its own (the memory-saving mode gathers x^T
    again in backward). Returns (codes [world, features, bytes], scales, handles)."""
    world = get_distributed_world_size(process_group)
    outs, handles = _gather_many_bytes(
        [data_t, scale_t_swz],
        [(world, data_t.shape[0], data_t.shape[1] * data_t.element_size()), (world * scale_t_swz.numel(),)],
        process_group, async_op)
    return outs[0], outs[1], handles
