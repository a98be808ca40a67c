"""Drop-in `Linear` with block-quantized forward, dgrad and wgrad GEMMs.

API, parameter naming, tensor-/sequence-parallel behaviour, the weight-quantization cache
across microbatches and the Megatron `main_grad` protocol follow the reference module
(miniTransformer/module/linear.py:27-949), so `class TELinear(Linear)` keeps working. What
is new underneath: the quantize backend in `QLinearParams.quantize_op` runs the sm_100a
kernels, sequence-parallel inputs can be gathered in quantized form (codes + scales, one
packed collective, after a MAX all-reduce of the per-tensor abs-max), and
`fuse_wgrad_accumulation` really accumulates into `weight.main_grad` in place.
"""
import contextlib
import logging
import os
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch

from . import config
from ._common import noop_cat
from .base import LayerLinearBaseModule
from ..distributed.distributed import (allreduce, gather_along_first_dim, gather_gemm_ready,
                                       gather_packed_along_first_dim, gather_transposed_as_k_slabs,
                                       get_distributed_rank, get_distributed_world_size,
                                       reduce_scatter_along_first_dim, set_tensor_model_parallel_attributes)
from ..ops import quantization
from ..utils.utils import cast_if_needed, divide, init_method_constant, is_rank_0

logger = logging.getLogger(__name__)

_NUM_FN_ARGS = 15


class _NonQuantizedLinear(torch.autograd.Function):
    """High-precision path: y = x w^T, dx = dy w, dw = dy^T x, with the same collectives."""

    @staticmethod
    def forward(ctx, x, x_meta, w, weight_qresult_cache, bias, sequence_parallel, tp_group, tp_size,
                parallel_mode, qlinear_params, activation_dtype, is_grad_enabled, is_first_microbatch,
                fuse_wgrad_accumulation, ub=None):
        x_shape = x.shape
        x = cast_if_needed(x.reshape(-1, x_shape[-1]), activation_dtype)
        bias = cast_if_needed(bias, activation_dtype)
        if parallel_mode == "column" and sequence_parallel:
            x, _ = gather_along_first_dim(x, tp_group)
        y = torch.nn.functional.linear(x, w, bias)
        if is_grad_enabled:
            ctx.use_bias = bias is not None
            ctx.sequence_parallel, ctx.tp_group, ctx.tp_size = sequence_parallel, tp_group, tp_size
            ctx.parallel_mode, ctx.x_shape = parallel_mode, x_shape
            ctx.save_for_backward(x, w)
        if parallel_mode == "row" and sequence_parallel:
            y, _ = reduce_scatter_along_first_dim(y, tp_group)
        elif parallel_mode == "row" and tp_size > 1:
            y, _ = allreduce(y, tp_group)
        return y.view(-1, *x_shape[1:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous().view(-1, dy.shape[-1])
        b_grad = dy.sum(dim=0) if ctx.use_bias else None
        if ctx.parallel_mode == "row" and ctx.sequence_parallel:
            dy, _ = gather_along_first_dim(dy, ctx.tp_group)
        dgrad = dy @ w
        handle = None
        if ctx.parallel_mode == "column" and ctx.sequence_parallel:
            dgrad, handle = reduce_scatter_along_first_dim(dgrad, ctx.tp_group, True)
        elif ctx.parallel_mode == "column" and ctx.tp_size > 1:
            dgrad, handle = allreduce(dgrad, ctx.tp_group, True)
        wgrad = dy.t() @ x
        if handle is not None:
            handle.wait()
        dgrad = dgrad.view(-1, *ctx.x_shape[1:])
        return (dgrad, None, wgrad, None, b_grad) + (None,) * (_NUM_FN_ARGS - 5)


def _overlap_sm_margin() -> int:
    """SMs the wgrad GEMM leaves to a collective that runs beside it (MT_TP_SM_MARGIN, default 16)."""
    try:
        return max(0, int(os.environ.get("MT_TP_SM_MARGIN", "16")))
    except ValueError:
        return 16


def _env_flag(name: str, default: bool) -> bool:
    v = os.environ.get(name)
    return default if v is None else v not in ("0", "")


def _sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count if torch.device(device).type == "cuda" else 0


def _margin_for(handles) -> int:
    """SMs a GEMM leaves idle for the exchanges behind `handles`: a resident GEMM CTA fills its
    SM (shared memory and registers), so a collective or copy kernel that should run beside the
    GEMM needs SMs of its own."""
    return _overlap_sm_margin() if any(getattr(h, "needs_sm_margin", True) for h in handles) else 0


def _sm_margin(op, sms: int):
    """Context in which the op's GEMMs leave `sms` SMs idle; ops without that control (the CPU
    stand-in of the tests) get a null context."""
    ctl = getattr(op, "sm_margin", None)
    return ctl(sms) if (ctl is not None and sms > 0) else contextlib.nullcontext()


def _gemm_opts(op, **kw):
    """Context with per-call GEMM options of the op's backend (ops without them: null context)."""
    ctl = getattr(op, "gemm_options", None)
    return ctl(**kw) if ctl is not None else contextlib.nullcontext()


def _peer_groups(ub, tp_group, device):
    """(peer group for gathers, peer group for reduce-scatters, buffer name, output meta) of a
    layer: peer-memory exchange is used when the layer was built with ub_overlap_ag /
    ub_overlap_rs and the group's ranks can share memory; otherwise None (process-group path)."""
    if ub is None:
        return None, None, "", None
    overlap_rs, overlap_ag, name, out_meta = ub
    pg = None
    if (overlap_rs or overlap_ag) and tp_group is not None and get_distributed_world_size(tp_group) > 1 \
            and _env_flag("MT_TP_PEER", True):
        from ..distributed.peer import get_peer_group
        pg = get_peer_group(tp_group, device)
    return (pg if overlap_ag else None), (pg if overlap_rs else None), name or "ub", out_meta


def _scatter_possible(pg, M, N, out_dtype, bias, world) -> bool:
    """The GEMM can push its output rows to the owning ranks: bf16 rows in slices of whole
    256-row tiles, a tile-kernel shape, and no bias inside the GEMM."""
    return (pg is not None and out_dtype == torch.bfloat16 and bias is None and M % (256 * world) == 0
            and N % 8 == 0 and N > 128 and M > 128)


def _scatter_is_link_bound(M, N, K, world) -> bool:
    """Whether a scattering GEMM spends more time pushing its output over NVLink (bf16 rows of the
    other ranks at about 600 GB/s) than computing (about 4.5 PFLOP/s): only then is there tensor
    time to give to a second GEMM running beside it."""
    link_s = M * N * 2.0 * (world - 1) / world / 600e9
    gemm_s = 2.0 * M * N * K / 4.5e15
    return link_s > 1.3 * gemm_s


def _gemm_reduce_scatter(pg, gemm, M, N, site, out_meta=None, defer=False):
    """Reduce-scatter of a GEMM's bf16 output along its rows, started by the GEMM itself:
    its epilogue stores every tile into the owning rank's staging buffer while later tiles are
    computed; after a barrier each rank sums the slices it received. With defer=True the
    barrier and the sum are returned as a callable, to be run after more work is enqueued."""
    from .. import kernels
    world = pg.world
    stage = pg.alternating(f"rs:{site}:{M}x{N}", M * N * 2)
    with kernels.gemm_options(scatter=(stage.ptrs, pg.rank, M // world)):
        gemm()

    def finish():
        pg.barrier()
        amax = None
        if out_meta is not None:
            amax = torch.zeros(1, dtype=torch.float32, device=pg.device)
            out_meta.amax = amax
        return pg.reduce_bf16(stage, M // world, N, amax)

    return finish if defer else finish()


def _interleave_gathered_transpose(stacked: torch.Tensor, world: int) -> torch.Tensor:
    """[world * R, C_local] (rank-major stack of per-rank transposed shards) -> [R, world * C_local]."""
    r = stacked.shape[0] // world
    return stacked.view(world, r, stacked.shape[1]).permute(1, 0, 2).reshape(r, world * stacked.shape[1])


class _QuantizedLinear(torch.autograd.Function):
    """Quantized path. All three GEMMs take K-major operands:
         fprop  y  = q(x)       . q(w)^T           contraction over in_features
         dgrad  dx = q(dy)      . q(w^T copy)^T    contraction over out_features
         wgrad  dw = q(dy^T copy) . q(x^T copy)^T  contraction over tokens (fp32 output)
    """

    @staticmethod
    def forward(ctx, x, x_meta, w, weight_qresult_cache, bias, sequence_parallel, tp_group, tp_size,
                parallel_mode, qlinear_params, activation_dtype, is_grad_enabled, is_first_microbatch,
                fuse_wgrad_accumulation, ub=None):
        """ub: None, or (overlap_rs, overlap_ag, name, out_meta) from a layer built with the
        userbuffer flags: the exchanges then run over peer memory (distributed/peer.py) where the
        shapes allow, else over the process group. out_meta (a QuantizeInputMeta or None)
        receives the abs-max of the output for the next layer's quantize."""
        op: quantization.QuantizeOpBase = qlinear_params.quantize_op
        assert op is not None, "QLinearParams.quantize_op is not set"
        x_shape = x.shape
        out_dtype = qlinear_params.mm_fprop.out_dtype or x.dtype
        x = cast_if_needed(x.reshape(-1, x_shape[-1]), activation_dtype)
        bias = cast_if_needed(bias, activation_dtype)

        gather_required = parallel_mode == "column" and sequence_parallel
        pg_ag, pg_rs, site, out_meta = _peer_groups(ub, tp_group, x.device)
        # the gather (when there is one, in its copy-free form) is left in flight while the weight
        # is quantized below, and awaited just before the GEMM
        qres_x = _QuantizedLinear.quantize_optionally_allgather(
            op, x, qlinear_params.x_params, transpose_required=is_grad_enabled,
            allgather_required=gather_required, allgather_quantize=qlinear_params.allgather_quantize,
            tp_group=tp_group, keep_transpose_local=qlinear_params.memory_saving and gather_required,
            weight_shape=tuple(w.shape), async_gather=True, input_meta=x_meta, peer_group=pg_ag, site=f"{site}:x")

        # weights are re-quantized on the first microbatch (or when the caller gives no hint),
        # unless the layer keeps its quantized weights until told to refresh them
        keep = bool(getattr(weight_qresult_cache, "keep", False)) and weight_qresult_cache.data is not None
        ready = getattr(weight_qresult_cache, "prefetched", None)
        if ready is not None and weight_qresult_cache.data is not None:
            # quantized ahead of this call on another stream (Linear.prefetch_quantized_weight)
            weight_qresult_cache.prefetched = None
            torch.cuda.current_stream().wait_event(ready)
            keep = True
        if not keep and (is_first_microbatch or is_first_microbatch is None or weight_qresult_cache.data is None):
            qres_w = op.quantize(w, qlinear_params.w_params, return_transpose=True)
            weight_qresult_cache.store(qres_w)
        else:
            qres_w = weight_qresult_cache.to_qresult()

        for h in getattr(qres_x, "_pending_handles", ()):
            h.wait()
        x_t_handles = getattr(qres_x, "_pending_handles_t", ())
        M, N = qres_x.data.shape[0], w.shape[0]
        scatter = (parallel_mode == "row" and sequence_parallel and
                   _scatter_possible(pg_rs, M, N, out_dtype, bias, get_distributed_world_size(tp_group)))
        amax_y = None
        if out_meta is not None and not scatter and (parallel_mode != "row" or tp_size == 1):
            amax_y = torch.zeros(1, dtype=torch.float32, device=x.device)

        def fprop():
            return op.qgemm(qres_x.data, qres_w.data, qlinear_params.mm_fprop, out_dtype, qres_x.scale, qres_w.scale,
                            bias, accumulate=False, global_amax_qx=qres_x.global_amax_row,
                            global_amax_qw=qres_w.global_amax_row, qparams_x=qlinear_params.x_params,
                            qparams_w=qlinear_params.w_params)

        # the gather of x^T (needed by wgrad only) may still be running: leave it SMs
        with _sm_margin(op, _margin_for(x_t_handles)):
            if scatter:
                y = _gemm_reduce_scatter(pg_rs, fprop, M, N, f"{site}:y", out_meta)
            elif amax_y is not None:
                with _gemm_opts(op, d_amax=amax_y):
                    y = fprop()
                out_meta.amax = amax_y
            else:
                y = fprop()
        if not is_grad_enabled:
            for h in x_t_handles:
                h.wait()

        if is_grad_enabled:
            ctx.use_bias = bias is not None
            ctx.sequence_parallel, ctx.tp_group, ctx.tp_size = sequence_parallel, tp_group, tp_size
            ctx.tp_rank = get_distributed_rank(tp_group)
            ctx.x_gather_required = gather_required
            ctx.parallel_mode, ctx.x_shape = parallel_mode, x_shape
            ctx.qlinear_params, ctx.quantize_op = qlinear_params, op
            ctx.is_first_microbatch = is_first_microbatch
            ctx.fuse_wgrad_accumulation = fuse_wgrad_accumulation
            ctx.activation_dtype = activation_dtype
            ctx.ub = ub
            ctx.x_t_is_local_shard = bool(getattr(qres_x, "_t_is_local_shard", False))
            ctx.x_t_handles = x_t_handles          # awaited in backward, before wgrad reads x^T
            ctx.x_t_sources = getattr(qres_x, "_pending_sources", None)
            # transposed copies only; their GEMM-layout scales travel as plain attributes
            ctx.sx_t_swz, ctx.sw_t_swz = qres_x.scale_t_swz, qres_w.scale_t_swz
            ctx.save_for_backward(qres_x.data_t, qres_x.scale_t, qres_x.global_amax_col,
                                  qres_w.data_t, qres_w.scale_t, qres_w.global_amax_col, w)

        if scatter:
            pass                                   # already reduced and scattered
        elif parallel_mode == "row" and sequence_parallel:
            y, _ = reduce_scatter_along_first_dim(y, tp_group)
        elif parallel_mode == "row" and tp_size > 1:
            y, _ = allreduce(y, tp_group)
        return y.view(-1, *x_shape[1:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        qx_t, sx_t, amax_x_col, qw_t, sw_t, amax_w_col, w = ctx.saved_tensors
        p, op = ctx.qlinear_params, ctx.quantize_op
        if sx_t is not None and ctx.sx_t_swz is not None:
            sx_t._mt_swz = ctx.sx_t_swz
        if ctx.sw_t_swz is not None:
            sw_t._mt_swz = ctx.sw_t_swz
        out_dtype_dgrad = p.mm_dgrad.out_dtype or dy.dtype
        dy = dy.contiguous().view(-1, dy.shape[-1])
        # the bias gradient (column sums of dy) comes out of the abs-max pass that quantizing dy
        # needs anyway, where the backend has such a pass; otherwise from a reduction of its own
        dy_meta = None
        if ctx.use_bias and dy.is_cuda and dy.dtype == torch.bfloat16:
            dy_meta = quantization.QuantizeInputMeta(col_sum=torch.empty(dy.shape[1], dtype=torch.float32, device=dy.device))

        gather_required = ctx.parallel_mode == "row" and ctx.sequence_parallel
        pg_ag, pg_rs, site, _ = _peer_groups(ctx.ub, ctx.tp_group, dy.device)
        qres_dy = _QuantizedLinear.quantize_optionally_allgather(
            op, dy, p.g_params, transpose_required=True, allgather_required=gather_required,
            allgather_quantize=p.allgather_quantize, tp_group=ctx.tp_group, weight_shape=tuple(w.shape),
            async_gather=True, input_meta=dy_meta, peer_group=pg_ag, site=f"{site}:dy")
        b_grad = None
        if ctx.use_bias:
            b_grad = dy_meta.col_sum.to(dy.dtype) if (dy_meta is not None and dy_meta.col_sum_done) else dy.sum(dim=0)
        for h in getattr(qres_dy, "_pending_handles", ()):
            h.wait()
        dy_t_handles = getattr(qres_dy, "_pending_handles_t", ())

        # memory-saving mode kept only this rank's token shard of x^T: gather it back while
        # the dgrad GEMM runs
        pending_x_t = None
        if ctx.x_t_is_local_shard:
            pending_x_t = _QuantizedLinear._start_gather_transposed(qx_t, sx_t, ctx.tp_group)

        M, N = qres_dy.data.shape[0], qw_t.shape[0]
        scatter = (ctx.parallel_mode == "column" and ctx.sequence_parallel and
                   _scatter_possible(pg_rs, M, N, out_dtype_dgrad, None, get_distributed_world_size(ctx.tp_group)))

        def dgrad_gemm():
            return op.qgemm(qres_dy.data, qw_t, p.mm_dgrad, out_dtype_dgrad, qres_dy.scale, sw_t, None, None,
                            accumulate=False, global_amax_qx=qres_dy.global_amax_row, global_amax_qw=amax_w_col,
                            qparams_x=p.g_params, qparams_w=p.w_params)

        def run_wgrad(margin):
            if ctx.is_first_microbatch is not None:
                accumulate = ctx.fuse_wgrad_accumulation and not ctx.is_first_microbatch
            else:
                accumulate = ctx.fuse_wgrad_accumulation
            main_grad = w.main_grad if ctx.fuse_wgrad_accumulation else None
            with _sm_margin(op, margin):
                return op.qgemm(qres_dy.data_t, qx_t_box[0], p.mm_wgrad,
                                # without main_grad: the parameter's type, what autograd would cast an
                                # fp32 gradient to (one rounding of the fp32 accumulator either way)
                                main_grad.dtype if main_grad is not None else (p.mm_wgrad.out_dtype or w.dtype),
                                qres_dy.scale_t, qx_t_box[1], None, out=main_grad, accumulate=accumulate,
                                global_amax_qx=qres_dy.global_amax_col, global_amax_qw=amax_x_col,
                                qparams_x=p.g_params, qparams_w=p.x_params)

        qx_t_box = [qx_t, sx_t]
        finish_dgrad, wgrad, handle = None, None, None
        late_handles = tuple(dy_t_handles) + tuple(getattr(ctx, "x_t_handles", ()))
        if (scatter and w.requires_grad and pending_x_t is None and _env_flag("MT_TP_CONCURRENT_WGRAD", True)
                and _scatter_is_link_bound(M, N, qres_dy.data.shape[1] * (2 if qres_dy.data.dtype == torch.uint8 else 1),
                                           get_distributed_world_size(ctx.tp_group))):
            # The dgrad GEMM that scatters its rows over NVLink is bound by the links, not by the
            # tensor cores: the wgrad GEMM runs beside it on a second stream, each on half of the
            # SMs, instead of behind it.
            for h in late_handles:
                h.wait()
            sms = _sm_count(dy.device)
            try:        # SMs of the scattering GEMM (MT_TP_SCATTER_SMS, default half); the wgrad GEMM takes the rest
                mine = min(sms - 8, max(8, int(os.environ.get("MT_TP_SCATTER_SMS", sms // 2)))) // 2 * 2
            except ValueError:
                mine = sms // 2
            box = []
            joined = pg_rs.on_side_stream(lambda: box.append(run_wgrad(mine)))
            with _sm_margin(op, sms - mine):
                finish_dgrad = _gemm_reduce_scatter(pg_rs, dgrad_gemm, M, N, f"{site}:dx", defer=True)
            joined.wait()
            wgrad = _QuantizedLinear.reset_wgrad_if_needed(ctx, w, box[0])
        else:
            # a gather of dy^T or of x^T (memory-saving mode) may be in flight: leave it SMs
            with _sm_margin(op, _overlap_sm_margin() if pending_x_t is not None else _margin_for(dy_t_handles)):
                if scatter:
                    # the tiles travel to their owners while the GEMM runs; the barrier and the local
                    # sum wait until the wgrad GEMM has been enqueued behind it
                    finish_dgrad = _gemm_reduce_scatter(pg_rs, dgrad_gemm, M, N, f"{site}:dx", defer=True)
                    dgrad = None
                else:
                    dgrad = dgrad_gemm()
            for h in late_handles:
                h.wait()

            if pending_x_t is not None:
                qx_t_box[0], qx_t_box[1] = _QuantizedLinear._finish_gather_transposed(pending_x_t, ctx.tp_group)

            if scatter:
                pass
            elif ctx.parallel_mode == "column" and ctx.sequence_parallel:
                dgrad, handle = reduce_scatter_along_first_dim(dgrad, ctx.tp_group, True)
            elif ctx.parallel_mode == "column" and ctx.tp_size > 1:
                dgrad, handle = allreduce(dgrad, ctx.tp_group, True)

            if w.requires_grad:
                # a reduce-scatter / all-reduce of dgrad is in flight: leave it SMs to run on
                wgrad = run_wgrad(_overlap_sm_margin() if handle is not None else 0)
                wgrad = _QuantizedLinear.reset_wgrad_if_needed(ctx, w, wgrad)

        if handle is not None:
            handle.wait()
        if finish_dgrad is not None:
            dgrad = finish_dgrad()
        dgrad = dgrad.view(-1, *ctx.x_shape[1:])
        return (dgrad, None, wgrad, None, b_grad) + (None,) * (_NUM_FN_ARGS - 5)

    # -- helpers ------------------------------------------------------------------------------
    @staticmethod
    def quantize_optionally_allgather(quantize_op, x, qparams, transpose_required, allgather_required,
                                      allgather_quantize, tp_group, keep_transpose_local=False, weight_shape=None,
                                      async_gather=False, input_meta=None, peer_group=None, site="ub"):
        """Quantizes x, gathering it across the tensor-parallel group first (bf16) or after
        (quantized) when the layer is sequence-parallel.

        Quantized gather: every rank quantizes its token shard with the MAX-all-reduced
        per-tensor abs-max, then ONE collective moves [codes | scales | codes^T | scales^T].
        Row-wise blocks run along features, so the gathered codes and scales are bit-identical
        to quantizing the gathered tensor. The transposed copy of each shard is a K-slice of
        the global transposed copy (shard length is a multiple of the block), re-interleaved
        after the gather."""
        if not allgather_required:
            return quantize_op.quantize(x, qparams, return_transpose=transpose_required, reduce_amax=False,
                                        tp_group=tp_group, input_meta=input_meta)
        assert tp_group is not None
        if not (allgather_quantize and quantize_op.supports_allgather):
            x, _ = gather_along_first_dim(x, tp_group)
            return quantize_op.quantize(x, qparams, return_transpose=transpose_required, reduce_amax=False,
                                        tp_group=tp_group)
        world = get_distributed_world_size(tp_group)
        block = qparams.quant_tile_shape[1] if qparams.quant_tile_shape else 32
        assert x.shape[0] % block == 0, "token shard must be a multiple of the quantization block"
        rows = x.shape[0]
        gather_t = transpose_required and not keep_transpose_local
        fmt = getattr(quantize_op, "format_name", None)
        if (peer_group is not None and fmt is not None and weight_shape is not None and min(weight_shape) > 128
                and _QuantizedLinear._gemm_ready_shapes(fmt, rows, x.shape[1], world, transpose_required)):
            return _QuantizedLinear._peer_gather_gemm_ready(peer_group, quantize_op, fmt, x, qparams, tp_group,
                                                            gather_t, transpose_required, input_meta, site)
        r = quantize_op.quantize(x, qparams, return_transpose=transpose_required, reduce_amax=True,
                                 tp_group=tp_group, input_meta=input_meta)
        if (weight_shape is not None and min(weight_shape) > 128
                and _QuantizedLinear._gemm_ready_gather_possible(r, rows, x.shape[1], world, transpose_required)):
            return _QuantizedLinear._gather_gemm_ready(r, tp_group, gather_t, transpose_required, async_gather)
        parts = [r.data, r.scale[:rows]]
        if gather_t:
            parts += [r.data_t, r.scale_t[: x.shape[1]]]
        g = gather_packed_along_first_dim(parts, tp_group)
        out = quantization.QuantizeResult(g[0], g[1], None, None, r.global_amax_row, r.global_amax_col)
        if gather_t:
            out.data_t = _interleave_gathered_transpose(g[2], world)
            out.scale_t = _interleave_gathered_transpose(g[3], world)
        elif transpose_required:
            out.data_t, out.scale_t = r.data_t, r.scale_t[: x.shape[1]]
            out._t_is_local_shard = True
        return out

    @staticmethod
    def _gemm_ready_shapes(fmt, rows, features, world, transpose_required):
        """Shape rules of the copy-free gather, known before anything is quantized: shards of
        whole 128-row scale chunks, K slabs of whole 128-byte K steps for the transposed copy
        (2 codes per byte in NVFP4), GEMM shapes the CTA-pair kernel takes."""
        if rows % 128 or rows * world <= 128 or features <= 128 or features % 128:
            return False
        t_row_bytes = rows // 2 if fmt == "nvfp4" else rows
        return not (transpose_required and t_row_bytes % 128)

    @staticmethod
    def _peer_gather_gemm_ready(pg, op, fmt, x, qparams, tp_group, gather_t, transpose_required, input_meta, site):
        """The copy-free quantized gather over peer memory: this rank's shard is quantized
        straight into its slot of a buffer every rank has mapped (with the abs-max MAX-reduced by
        a one-warp exchange first, where the format has one); after a barrier one copy kernel
        pulls the other ranks' row-wise codes and scales, and a second one, on a side stream,
        the transposed copies that only the wgrad GEMM needs."""
        from .. import kernels
        world, (rows, cols) = pg.world, x.shape
        sizes = kernels.quantized_shard_bytes(fmt, rows, cols)
        offs, total = [], 0
        for n in sizes:
            offs.append(total)
            total += (n + 255) // 256 * 256
        shared = pg.alternating(f"ag:{site}:{fmt}:{rows}x{cols}", total)
        keys = ("q", "s_swz", "q_t", "s_t_swz")
        into = {k: shared.tensor[o:o + n] for k, o, n in zip(keys, offs, sizes) if transpose_required or k in keys[:2]}
        meta = quantization.QuantizeInputMeta(
            amax=getattr(input_meta, "amax", None), amax_col=getattr(input_meta, "amax_col", None), into=into,
            amax_reduce=pg.allreduce_max_, col_sum=getattr(input_meta, "col_sum", None))
        r = op.quantize(x, qparams, return_transpose=transpose_required, reduce_amax=True, tp_group=tp_group,
                        input_meta=meta)
        if meta.col_sum_done:
            input_meta.col_sum_done = True
        pg.barrier()
        dev, u8 = x.device, torch.uint8
        data = torch.empty((world * rows, sizes[0] // rows), dtype=u8, device=dev)
        scale = torch.empty(world * sizes[1], dtype=u8, device=dev)
        # both pulls run on a side stream: the caller quantizes the weight meanwhile and waits for the
        # row-wise copy just before the GEMM that reads it
        segs_row = [(offs[0], data, sizes[0]), (offs[1], scale, sizes[1])]
        h_row = pg.on_side_stream(lambda: pg.gather(shared, segs_row), keep=(data, scale))
        if r.data.dtype != u8:
            data = data.view(r.data.dtype)
        scale._mt_swz = scale
        out = quantization.QuantizeResult(data, scale, None, None, r.global_amax_row, r.global_amax_col, scale, None)
        out._pending_handles = (h_row,)
        out._pending_handles_t = ()
        if gather_t:
            data_t = torch.empty((world, cols, sizes[2] // cols), dtype=u8, device=dev)
            scale_t = torch.empty(world * sizes[3], dtype=u8, device=dev)
            segs = [(offs[2], data_t, sizes[2]), (offs[3], scale_t, sizes[3])]
            out._pending_handles_t = (pg.on_side_stream(lambda: pg.gather(shared, segs, ctas=max(4, _overlap_sm_margin()) // 2 * 2, whole_sms=True), keep=(data_t, scale_t)),)
            if r.data_t.dtype != u8:
                data_t = data_t.view(r.data_t.dtype)
            scale_t._mt_swz = scale_t
            out.data_t, out.scale_t, out.scale_t_swz = data_t, scale_t, scale_t
        elif transpose_required:
            # memory-saving mode keeps this rank's shard of x^T until backward: out of the slot,
            # which later gathers rewrite
            s_t = r.scale_t.clone()
            s_t._mt_swz = r.scale_t_swz.clone()
            out.data_t, out.scale_t, out.scale_t_swz = r.data_t.clone(), s_t, s_t._mt_swz
            out._t_is_local_shard = True
        return out

    @staticmethod
    def _gemm_ready_gather_possible(r, rows, features, world, transpose_required):
        """The copy-free gather needs GEMM-layout scales from the quantizer, shards of whole
        128-row scale chunks, K slabs of whole 128-byte K steps for the transposed copy, and
        GEMM shapes the CTA-pair kernel takes (more than 128 rows on both sides)."""
        if r.scale_swz is None or (transpose_required and r.scale_t_swz is None):
            return False
        if rows % 128 or rows * world <= 128 or features <= 128:
            return False
        if transpose_required and (r.data_t.shape[1] * r.data_t.element_size()) % 128:
            return False
        return True

    @staticmethod
    def _gather_gemm_ready(r, tp_group, gather_t, transpose_required, async_gather=False):
        """Quantized gather without any copy after the collectives: row-wise codes and
        GEMM-layout scales land where the fprop / dgrad GEMM reads them; the transposed copies
        stay per-rank K slabs ([world, features, bytes]) that the wgrad GEMM walks slab by slab.
        The scale fields of the result hold the GEMM layout (the row-major form is not
        materialized on this path)."""
        handles_t = ()
        async_gather = async_gather and _env_flag("MT_TP_ASYNC_GATHER", True)
        # Splitting pays on 2 ranks (3.69 against 3.78 ms per step of the benchmark MLP); on 8 ranks
        # one collective awaited before the GEMM measured faster (1.85 against 2.16 ms), the extra
        # launches costing more there than the overlap returns.
        if async_gather and gather_t and _env_flag("MT_TP_SPLIT_GATHER", get_distributed_world_size(tp_group) <= 2):
            # two collectives: the row-wise copy is needed by the next GEMM (fprop / dgrad), the
            # transposed one only by wgrad, so it may stay in flight under that GEMM
            data, scale, _, _, handles = gather_gemm_ready(r.data, r.scale_swz, tp_group, async_op=True)
            data_t, scale_t, handles_t = gather_transposed_as_k_slabs(r.data_t, r.scale_t_swz, tp_group, async_op=True)
        else:
            data, scale, data_t, scale_t, handles = gather_gemm_ready(
                r.data, r.scale_swz, tp_group, r.data_t if gather_t else None, r.scale_t_swz if gather_t else None,
                async_op=async_gather)
        if r.data.dtype != torch.uint8:
            data = data.view(r.data.dtype)
        scale._mt_swz = scale
        out = quantization.QuantizeResult(data, scale, None, None, r.global_amax_row, r.global_amax_col, scale, None)
        if async_gather:
            # the caller waits on these before the first use of the gathered tensors; the sources
            # stay referenced until then
            out._pending_handles = tuple(handles)
            out._pending_handles_t = tuple(handles_t)
            out._pending_sources = (r.data, r.scale_swz, r.data_t, r.scale_t_swz)
        if gather_t:
            if r.data_t.dtype != torch.uint8:
                data_t = data_t.view(r.data_t.dtype)
            scale_t._mt_swz = scale_t
            out.data_t, out.scale_t, out.scale_t_swz = data_t, scale_t, scale_t
        elif transpose_required:
            out.data_t, out.scale_t, out.scale_t_swz = r.data_t, r.scale_t, r.scale_t_swz
            out._t_is_local_shard = True
        return out

    @staticmethod
    def _start_gather_transposed(qx_t, sx_t, tp_group):
        world = get_distributed_world_size(tp_group)
        swz = getattr(sx_t, "_mt_swz", None)
        if swz is not None and (qx_t.shape[1] * qx_t.element_size()) % 128 == 0 and qx_t.shape[0] > 128:
            data_t, scale_t, handles = gather_transposed_as_k_slabs(qx_t, swz, tp_group, async_op=True)
            if qx_t.dtype != torch.uint8:
                data_t = data_t.view(qx_t.dtype)
            return ("slabs", data_t, scale_t, handles)
        flat = torch.cat([qx_t.contiguous().view(torch.uint8).reshape(-1),
                          sx_t.contiguous().view(torch.uint8).reshape(-1)])
        out = torch.empty(world * flat.numel(), dtype=torch.uint8, device=flat.device)
        handle = torch.distributed.all_gather_into_tensor(out, flat, group=tp_group, async_op=True)
        return out, handle, qx_t, sx_t

    @staticmethod
    def _finish_gather_transposed(pending, tp_group):
        if pending[0] == "slabs":
            _, data_t, scale_t, handles = pending
            for h in handles:
                if h is not None:
                    h.wait()
            scale_t._mt_swz = scale_t
            return data_t, scale_t
        out, handle, qx_t, sx_t = pending
        handle.wait()
        world = get_distributed_world_size(tp_group)
        out = out.view(world, -1)
        nq = qx_t.numel() * qx_t.element_size()   # bytes of the codes inside each rank's packet

        def unpack(piece, like):
            flat = piece.contiguous().reshape(-1)
            if like.dtype != torch.uint8:
                flat = flat.view(like.dtype)
            return _interleave_gathered_transpose(flat.reshape(world * like.shape[0], like.shape[1]), world)

        return unpack(out[:, :nq], qx_t), unpack(out[:, nq:], sx_t)

    @staticmethod
    def reset_wgrad_if_needed(ctx, w, wgrad):
        """Megatron's main_grad protocol (miniTransformer/module/linear.py:515-550): once the
        gradient sits in w.main_grad, autograd gets a dummy of the weight's shape (zeros when
        the parameter asks for it) or nothing at all."""
        if not w.requires_grad:
            return None
        if not ctx.fuse_wgrad_accumulation:
            return wgrad
        if hasattr(w, "grad_added_to_main_grad"):
            make = torch.zeros if getattr(w, "zero_out_wgrad", False) else torch.empty
            w.grad_added_to_main_grad = True
            return make(w.main_grad.shape, dtype=w.dtype, device=w.device, requires_grad=False)
        return None


class Linear(LayerLinearBaseModule):
    """y = x A^T + b with optional block-quantized GEMMs; drop-in for `torch.nn.Linear` /
    TransformerEngine's `Linear` (constructor and forward signature of
    miniTransformer/module/linear.py:632-655, 864-870).

    parallel_mode: None | "column" | "row" (Megatron tensor parallelism; `in_features` /
    `out_features` are divided accordingly). sequence_parallel: all-gather before a column
    layer, reduce-scatter after a row layer. fuse_wgrad_accumulation: accumulate the weight
    gradient into `weight.main_grad`. return_bias: hand the bias back instead of adding it.
    parameters_split: names (or name -> size) of several parameters carved out of one weight
    buffer along dim 0. qlinear_params: the recipe; if None it is taken from QAT_PARAMS.
    """

    def __init__(self, in_features: int, out_features: int, sequence_parallel: bool = False,
                 fuse_wgrad_accumulation: bool = False, tp_group=None, tp_size: int = 1,
                 get_rng_state_tracker: Optional[Callable] = None, rng_tracker_name: Optional[str] = None,
                 init_method: Optional[Callable] = None, bias: bool = True, return_bias: bool = False,
                 params_dtype: Optional[torch.dtype] = None, parallel_mode: Optional[str] = None,
                 parameters_split: Optional[Union[Tuple[str, ...], Dict[str, int]]] = None,
                 device: Union[torch.device, str] = "cuda", ub_overlap_rs: bool = False,
                 ub_overlap_ag: bool = False, ub_name: Optional[str] = None,
                 layer_number: Optional[int] = None,
                 qlinear_params: Optional[config.QLinearParams] = None) -> None:
        super().__init__(tp_group, tp_size, sequence_parallel)
        params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        self.in_features, self.out_features = in_features, out_features
        self.fuse_wgrad_accumulation = fuse_wgrad_accumulation
        self.use_bias, self.return_bias = bias, return_bias
        self.apply_bias = bias and not return_bias
        self.ub_overlap_rs, self.ub_overlap_ag = ub_overlap_rs, ub_overlap_ag
        # ub_overlap_rs: the reduce-scatter after a row-parallel GEMM (and after the dgrad GEMM of a
        # column-parallel layer) is done by the GEMM's own epilogue over NVLink peer memory;
        # ub_overlap_ag: quantized activations are gathered by peer copies (distributed/peer.py)
        if ub_overlap_rs or ub_overlap_ag:
            assert ub_name is not None, "Userbuffer name [string] is not set."
        self.ub_name = self.layer_name = ub_name
        # emit_output_amax: the forward GEMM (or the reduce step after it) also computes max |y|;
        # `output_meta` then holds it for the next layer's `inp_meta` (no abs-max pass over y)
        self.emit_output_amax = False
        self.output_meta: Optional[quantization.QuantizeInputMeta] = None
        self.get_rng_state_tracker, self.rng_tracker_name = get_rng_state_tracker, rng_tracker_name
        self.layer_number = layer_number
        self.qlinear_params = self.set_qlinear_params(qlinear_params=qlinear_params, layer_number=layer_number,
                                                      layer_name=self.layer_name)
        if is_rank_0():
            logger.info("layer %s linear %s uses %s", layer_number, self.layer_name, self.qlinear_params)
        if device == "meta":
            assert parameters_split is None, "Cannot split module parameters on 'meta' device."
        assert parallel_mode in ("row", "column", None), f"parallel_mode {parallel_mode} not supported"
        self.parallel_mode = parallel_mode
        if self.tp_size > 1 and torch.cuda.is_available():
            # The tensor-parallel paths run gathers, weight quantization and wgrad GEMMs on side
            # streams with grids sized to share the SMs with the main stream's kernels; kernels
            # that become resident ahead of their turn would take those SMs (the 8-rank MLP step
            # measured slower with early launches than in the runs before they existed).
            from .. import kernels
            kernels.set_launch_overlap(False)
        if parallel_mode == "column":
            self.out_features = divide(out_features, self.tp_size)
        elif parallel_mode == "row":
            self.in_features = divide(in_features, self.tp_size)

        weight_buf = torch.empty(self.out_features, self.in_features, device=device, dtype=params_dtype)
        bias_buf = torch.empty(self.out_features, device=device, dtype=params_dtype) if bias else None

        # names and sizes of the parameters carved out of the buffers
        if parameters_split is None:
            names, sizes = [""], [out_features]
        elif not parameters_split:
            raise ValueError("Cannot split weight buffer into 0 parameters")
        elif isinstance(parameters_split, dict):
            names, sizes = [n.rstrip("_") for n in parameters_split], list(parameters_split.values())
        elif all(isinstance(n, str) for n in parameters_split):
            assert out_features % len(parameters_split) == 0, "Invalid split size"
            names = [n.rstrip("_") for n in parameters_split]
            sizes = [out_features // len(names)] * len(names)
        else:
            raise TypeError("Invalid configuration for parameters split")
        if sum(sizes) != out_features:
            raise ValueError(f"Trying to split weight buffer ({out_features=}) with split sizes {sizes}")
        if parallel_mode == "column":
            for s in sizes:
                if s % self.tp_size != 0:
                    raise RuntimeError(f"Attempting to distribute a parameter with out_features={s} "
                                       f"between {self.tp_size} tensor-parallel processes")
            sizes = [s // self.tp_size for s in sizes]
        self.weight_names = [f"{n}_weight" if n else "weight" for n in names]
        self.bias_names = [f"{n}_bias" if n else "bias" for n in names]
        self.parameter_split_sizes = sizes

        # weights first, so they stay adjacent in parameters(); then biases
        off = 0
        for name, size in zip(self.weight_names, sizes):
            self.register_parameter(name, torch.nn.Parameter(weight_buf[off:off + size]), init_fn=init_method,
                                    get_rng_state_tracker=get_rng_state_tracker)
            off += size
        off = 0
        for name, size in zip(self.bias_names, sizes):
            if bias:
                self.register_parameter(name, torch.nn.Parameter(bias_buf[off:off + size]),
                                        init_fn=init_method_constant(0.0))
            else:
                setattr(self, name, torch.empty(0, dtype=params_dtype, device=device))
            off += size

        self.reset_parameters(defer_init=(device == "meta"))
        self.weight_qresult_cache = quantization.QuantizeResultCache()
        # a row-parallel bias can only be added after the collective
        self.gemm_bias_unfused_add = parallel_mode == "row" and self.apply_bias

    _prefetch_streams: Dict[int, "torch.cuda.Stream"] = {}

    def prefetch_quantized_weight(self) -> None:
        """Quantizes the current weight now, on a side stream, for the next forward call, which
        then uses these copies instead of quantizing on its own stream (whatever
        is_first_microbatch says). A training loop calls it for the layers of a block once the
        optimizer has updated them, e.g. at the start of the step: the quantize passes of all
        weights then run beside the first layers' activation work instead of between their
        GEMMs."""
        if not self.qlinear_params.quantize:
            return
        weight = noop_cat([getattr(self, n) for n in self.weight_names]).detach()
        dev = weight.device
        side = Linear._prefetch_streams.get(dev.index)
        if side is None:
            side = Linear._prefetch_streams[dev.index] = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            q = self.qlinear_params.quantize_op.quantize(weight, self.qlinear_params.w_params, return_transpose=True)
            ev = torch.cuda.Event()
            ev.record(side)
        if not torch.cuda.is_current_stream_capturing():
            for t in (q.data, q.scale, q.data_t, q.scale_t, q.global_amax_row, q.global_amax_col, q.scale_swz,
                      q.scale_t_swz):
                if t is not None:
                    t.record_stream(main)      # produced on the side stream, consumed on this one
        self.weight_qresult_cache.store(q)
        self.weight_qresult_cache.prefetched = ev

    def reset_parameters(self, defer_init=False):
        super().reset_parameters(defer_init=defer_init)
        if defer_init:
            return
        for name in self.weight_names:
            set_tensor_model_parallel_attributes(getattr(self, name), True, 1 if self.parallel_mode == "row" else 0, 1)
        if self.use_bias:
            for name in self.bias_names:
                if self.parallel_mode == "row":
                    getattr(self, name).sequence_parallel = self.sequence_parallel
                elif self.parallel_mode == "column":
                    set_tensor_model_parallel_attributes(getattr(self, name), True, 0, 1)

    @torch._dynamo.disable(recursive=True)
    def forward(self, inp: torch.Tensor, is_first_microbatch: Optional[bool] = None,
                fp8_output: Optional[bool] = False,
                inp_meta: Optional[quantization.QuantizeInputMetaBase] = None):
        """is_first_microbatch: True / False let the layer cache the quantized weight across
        the microbatches of a step and skip the wgrad accumulation on the first one; None
        re-quantizes every call."""
        self.set_activation_dtype(inp)
        inp = inp.contiguous()
        assert self.tp_group_initialized, "TP group not initialized"
        assert inp.dtype in (torch.float32, torch.float16, torch.bfloat16), f"Input dtype {inp.dtype} not supported"
        assert fp8_output is False, "FP8 output is not supported yet"

        weight = noop_cat([getattr(self, n) for n in self.weight_names])
        bias = noop_cat([getattr(self, n) for n in self.bias_names]) if self.use_bias else getattr(self, self.bias_names[0])

        fn = _QuantizedLinear if self.qlinear_params.quantize else _NonQuantizedLinear
        grad = torch.is_grad_enabled()
        args: List[Any] = [] if grad else [None]
        args += [inp, inp_meta, weight, self.weight_qresult_cache,
                 bias if self.apply_bias and not self.gemm_bias_unfused_add else None,
                 self.sequence_parallel, self.tp_group, self.tp_size, self.parallel_mode, self.qlinear_params,
                 self.activation_dtype, grad, is_first_microbatch, self.fuse_wgrad_accumulation]
        self.weight_qresult_cache.keep = bool(self.primary_weights_in_fp8)
        self.output_meta = quantization.QuantizeInputMeta() if self.emit_output_amax else None
        ub = None
        if self.ub_overlap_rs or self.ub_overlap_ag or self.output_meta is not None:
            ub = (self.ub_overlap_rs, self.ub_overlap_ag, self.ub_name, self.output_meta)
        args.append(ub)
        out = (fn.apply if grad else fn.forward)(*args)
        if self.gemm_bias_unfused_add:
            out = out + cast_if_needed(bias, self.activation_dtype)
        if self.return_bias:
            return out, cast_if_needed(bias, self.activation_dtype)
        return out
