"""GroupedLinear: one linear layer per expert applied to consecutive row groups of the input
(MoE expert GEMMs), block-quantized with the MXFP8 backend.

API and parameter naming (`weight{i}`, `bias{i}`, `forward(inp, m_splits,
is_first_microbatch)`, `out_features % 128 == 0`, no sequence parallelism, all-reduce for
tensor parallelism, per-group bias added outside the GEMM) follow the reference module
(miniTransformer/module/group_linear.py:33-513). The reference file cannot be imported and
its arithmetic callees do not exist; the arithmetic here is the MXFP8 recipe on the sm_100a
grouped kernels:
  fprop  y[rows of g]  = q(x)[rows of g] . q(w_g)^T
  dgrad  dx[rows of g] = q(dy)[rows of g] . q(w_g^T)^T
  wgrad  dw_g          = q(dy_g^T) . q(x_g^T)^T   with 1x32 blocks restarting at each group.
"""
import logging
from typing import Callable, List, Optional, Tuple, Union

import torch

from . import config
from ._common import stacked_view
from .base import LayerLinearBaseModule
from ..distributed.distributed import allreduce, get_distributed_rank, set_tensor_model_parallel_attributes
from ..ops import quantization
from ..utils.utils import cast_if_needed, divide, init_method_constant, is_rank_0

logger = logging.getLogger(__name__)

_NUM_FIXED_ARGS = 11


class _QuantizedGroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, m_splits, weight_qresult_cache, tp_group, tp_size, parallel_mode, qlinear_params,
                activation_dtype, is_grad_enabled, is_first_microbatch, fuse_wgrad_accumulation, *weights):
        op = qlinear_params.quantize_op
        assert op is not None and hasattr(op, "grouped_qgemm"), "the recipe's backend has no grouped operations"
        x_shape = x.shape
        out_dtype = qlinear_params.mm_fprop.out_dtype or x.dtype
        x = cast_if_needed(x.reshape(-1, x_shape[-1]), activation_dtype)
        G, (N, K) = len(weights), weights[0].shape

        # With a backend that can do it, the per-group transposed copy that wgrad contracts over
        # is produced by the same pass over x (and saved instead of x itself: 1 byte per element
        # instead of 2); otherwise x is saved and transposed in backward.
        fused_t = is_grad_enabled and hasattr(op, "grouped_quantize_with_transpose") and \
            any(w.requires_grad for w in weights)
        x_t = None
        if fused_t:
            qres_x, x_t = op.grouped_quantize_with_transpose(x, qlinear_params.x_params, m_splits)
        else:
            qres_x = op.quantize(x, qlinear_params.x_params, return_transpose=False)
        # (a cache filled under no_grad holds no transposed copy: refill it before a training pass)
        if (is_first_microbatch or is_first_microbatch is None or weight_qresult_cache.data is None
                or (is_grad_enabled and weight_qresult_cache.data_t is None)):
            # expert weights allocated by this module sit back to back: no stacking copy
            w_all = stacked_view(weights)
            if w_all is None:
                w_all = torch.stack(weights, dim=0)
            qres_w = op.grouped_quantize(w_all, qlinear_params.w_params, return_transpose=is_grad_enabled)
            weight_qresult_cache.store(qres_w)
        else:
            qres_w = weight_qresult_cache.to_qresult()

        y = op.grouped_qgemm(qres_x.data, qres_w.data, qlinear_params.mm_fprop, out_dtype, qres_x.scale,
                             qres_w.scale, m_splits=m_splits, biases=None, qparams_x=qlinear_params.x_params,
                             qparams_w=qlinear_params.w_params, weights_transposed=False, n_out=N)

        if is_grad_enabled:
            ctx.m_splits, ctx.tp_group, ctx.tp_size = list(m_splits), tp_group, tp_size
            ctx.parallel_mode, ctx.x_shape = parallel_mode, x_shape
            ctx.qlinear_params, ctx.quantize_op = qlinear_params, op
            ctx.is_first_microbatch, ctx.fuse_wgrad_accumulation = is_first_microbatch, fuse_wgrad_accumulation
            ctx.num_gemms, ctx.in_features = G, K
            ctx.sw_t_swz = qres_w.scale_t_swz
            ctx.weights = weights
            ctx.x_t_pad = x_t[2] if x_t is not None else None
            if x_t is not None:
                ctx.save_for_backward(None, qres_w.data_t, qres_w.scale_t, x_t[0], x_t[1])
            else:
                ctx.save_for_backward(x, qres_w.data_t, qres_w.scale_t, None, None)

        if parallel_mode == "row" and tp_size > 1:
            y, _ = allreduce(y, tp_group)
        return y.view(-1, *x_shape[1:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x, qw_t, sw_t, x_t_q, x_t_s = ctx.saved_tensors
        p, op = ctx.qlinear_params, ctx.quantize_op
        if ctx.sw_t_swz is not None:
            sw_t._mt_swz = ctx.sw_t_swz
        out_dtype_dgrad = p.mm_dgrad.out_dtype or dy.dtype
        dy = dy.contiguous().view(-1, dy.shape[-1])

        need_wgrad = any(w.requires_grad for w in ctx.weights)
        dy_t = None
        if need_wgrad and hasattr(op, "grouped_quantize_with_transpose"):
            qres_dy, dy_t = op.grouped_quantize_with_transpose(dy, p.g_params, ctx.m_splits)
        else:
            qres_dy = op.quantize(dy, p.g_params, return_transpose=False)
        dgrad = op.grouped_qgemm(qres_dy.data, qw_t, p.mm_dgrad, out_dtype_dgrad, qres_dy.scale, sw_t,
                                 m_splits=ctx.m_splits, biases=None, qparams_x=p.g_params, qparams_w=p.w_params,
                                 weights_transposed=True, n_out=ctx.in_features)
        handle = None
        if ctx.parallel_mode == "column" and ctx.tp_size > 1:
            dgrad, handle = allreduce(dgrad, ctx.tp_group, True)

        wgrads: List[Optional[torch.Tensor]] = [None] * ctx.num_gemms
        if need_wgrad:
            if dy_t is None:
                dy_t = op.grouped_transpose_quantize(dy, ctx.m_splits)
            x_t = (x_t_q, x_t_s, ctx.x_t_pad) if x_t_q is not None else op.grouped_transpose_quantize(x, ctx.m_splits)
            accumulate = ctx.fuse_wgrad_accumulation and (ctx.is_first_microbatch is None or not ctx.is_first_microbatch)
            # Output type: the main_grad type when accumulating there; otherwise the parameter
            # type, which is what autograd would cast an fp32 gradient to (one rounding of the
            # fp32 accumulator either way), unless the recipe names a type.
            main_all = None
            if ctx.fuse_wgrad_accumulation:
                out_dtype_wgrad = ctx.weights[0].main_grad.dtype
                if all(w.requires_grad for w in ctx.weights):
                    main_all = stacked_view([w.main_grad for w in ctx.weights])
            else:
                out_dtype_wgrad = p.mm_wgrad.out_dtype or ctx.weights[0].dtype
            if main_all is not None:
                # main_grad buffers sit back to back: the GEMM writes (or accumulates) in place
                wg = op.grouped_gemm_1d1d(dy_t, x_t, out_dtype_wgrad, single_output=True, out=main_all,
                                          accumulate=accumulate)
            else:
                wg = op.grouped_gemm_1d1d(dy_t, x_t, out_dtype_wgrad, single_output=True)
            for i, w in enumerate(ctx.weights):
                if not w.requires_grad:
                    continue
                if ctx.fuse_wgrad_accumulation:
                    # Megatron main_grad protocol, per expert
                    if main_all is not None:
                        pass
                    elif accumulate:
                        w.main_grad.add_(wg[i])
                    else:
                        w.main_grad.copy_(wg[i])
                    if hasattr(w, "grad_added_to_main_grad"):
                        w.grad_added_to_main_grad = True
                        make = torch.zeros if getattr(w, "zero_out_wgrad", False) else torch.empty
                        wgrads[i] = make(w.shape, dtype=w.dtype, device=w.device)
                else:
                    wgrads[i] = wg[i]
        if handle is not None:
            handle.wait()
        return (dgrad.view(-1, *ctx.x_shape[1:]),) + (None,) * (_NUM_FIXED_ARGS - 1) + tuple(wgrads)


class _NonQuantizedGroupedLinear(torch.autograd.Function):
    """bf16 path: per-group torch matmuls (used by the non-quantized recipe)."""

    @staticmethod
    def forward(ctx, x, m_splits, weight_qresult_cache, tp_group, tp_size, parallel_mode, qlinear_params,
                activation_dtype, is_grad_enabled, is_first_microbatch, fuse_wgrad_accumulation, *weights):
        x_shape = x.shape
        x = cast_if_needed(x.reshape(-1, x_shape[-1]), activation_dtype)
        ys = [xs @ w.t() for xs, w in zip(torch.split(x, list(m_splits)), weights)]
        y = torch.cat(ys) if ys else x.new_zeros((0, weights[0].shape[0]))
        if is_grad_enabled:
            ctx.m_splits, ctx.tp_group, ctx.tp_size, ctx.parallel_mode, ctx.x_shape = list(m_splits), tp_group, tp_size, parallel_mode, x_shape
            ctx.save_for_backward(x, *weights)
        if parallel_mode == "row" and tp_size > 1:
            y, _ = allreduce(y, tp_group)
        return y.view(-1, *x_shape[1:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x, *weights = ctx.saved_tensors
        dy = dy.contiguous().view(-1, dy.shape[-1])
        dys, xs = torch.split(dy, ctx.m_splits), torch.split(x, ctx.m_splits)
        dgrad = torch.cat([d @ w for d, w in zip(dys, weights)])
        if ctx.parallel_mode == "column" and ctx.tp_size > 1:
            dgrad, _ = allreduce(dgrad, ctx.tp_group)
        wgrads = tuple(d.t() @ xx for d, xx in zip(dys, xs))
        return (dgrad.view(-1, *ctx.x_shape[1:]),) + (None,) * (_NUM_FIXED_ARGS - 1) + wgrads


class GroupedLinear(LayerLinearBaseModule):
    """`num_gemms` independent linear layers; `forward(inp, m_splits)` applies layer i to the
    i-th group of `m_splits[i]` consecutive rows of `inp`. Constructor arguments as in `Linear`
    (without `parameters_split`); parameters are `weight{i}` [out, in] and `bias{i}`."""

    def __init__(self, num_gemms: int, in_features: int, out_features: int, sequence_parallel: bool = False,
                 fuse_wgrad_accumulation: bool = False, tp_group=None, tp_size: int = 1,
                 get_rng_state_tracker: Optional[Callable] = None, rng_tracker_name: Optional[str] = None,
                 init_method: Optional[Callable] = None, bias: bool = True, return_bias: bool = False,
                 params_dtype: Optional[torch.dtype] = None, parallel_mode: Optional[str] = None,
                 device: Union[torch.device, str] = "cuda", ub_overlap_rs: bool = False, ub_overlap_ag: bool = False,
                 ub_name: Optional[str] = None, layer_number: Optional[int] = None,
                 qlinear_params: Optional[config.QLinearParams] = None) -> None:
        super().__init__(tp_group, tp_size, sequence_parallel)
        params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        self.num_gemms = num_gemms
        self.in_features, self.out_features = in_features, out_features
        self.fuse_wgrad_accumulation = fuse_wgrad_accumulation
        self.use_bias, self.return_bias = bias, return_bias
        self.apply_bias = bias and not return_bias
        self.ub_name = self.layer_name = ub_name
        self.get_rng_state_tracker, self.rng_tracker_name = get_rng_state_tracker, rng_tracker_name
        self.layer_number = layer_number
        assert not self.sequence_parallel, "GroupedLinear does not support sequence parallelism"
        assert parallel_mode in ("row", "column", None), f"parallel_mode {parallel_mode} not supported"
        self.parallel_mode = parallel_mode
        if parallel_mode == "column":
            self.out_features = divide(out_features, self.tp_size)
        elif parallel_mode == "row":
            self.in_features = divide(in_features, self.tp_size)
        assert self.out_features % 128 == 0 and self.in_features % 128 == 0, \
            "GroupedLinear needs in/out features that are multiples of 128"
        self.qlinear_params = self.set_qlinear_params(qlinear_params=qlinear_params, layer_number=layer_number,
                                                      layer_name=self.layer_name)
        if is_rank_0():
            logger.info("layer %s grouped linear %s (%d experts) uses %s", layer_number, self.layer_name, num_gemms,
                        self.qlinear_params)
        # All expert weights live in one block, each `weight{i}` a view of it, so that the
        # grouped quantize reads them as one [num_gemms, out, in] tensor without a stacking copy.
        block = torch.empty(num_gemms, self.out_features, self.in_features, device=device, dtype=params_dtype)
        for i in range(num_gemms):
            self.register_parameter(f"weight{i}", torch.nn.Parameter(block[i]),
                                    init_fn=init_method, get_rng_state_tracker=get_rng_state_tracker)
            if bias:
                self.register_parameter(f"bias{i}", torch.nn.Parameter(
                    torch.empty(self.out_features, device=device, dtype=params_dtype)), init_fn=init_method_constant(0.0))
            else:
                setattr(self, f"bias{i}", torch.empty(0, dtype=params_dtype, device=device))
        self.reset_parameters(defer_init=(device == "meta"))
        self.weight_qresult_cache = quantization.QuantizeResultCache()
        # the bias is always added per group after the GEMM
        self.gemm_bias_unfused_add = self.apply_bias

    def reset_parameters(self, defer_init=False):
        super().reset_parameters(defer_init=defer_init)
        if defer_init:
            return
        for i in range(self.num_gemms):
            set_tensor_model_parallel_attributes(getattr(self, f"weight{i}"), True,
                                                 1 if self.parallel_mode == "row" else 0, 1)
            if self.use_bias:
                if self.parallel_mode == "row":
                    getattr(self, f"bias{i}").sequence_parallel = self.sequence_parallel
                elif self.parallel_mode == "column":
                    set_tensor_model_parallel_attributes(getattr(self, f"bias{i}"), True, 0, 1)

    @torch._dynamo.disable(recursive=True)
    def forward(self, inp: torch.Tensor, m_splits: List[int], is_first_microbatch: Optional[bool] = None):
        assert len(m_splits) == self.num_gemms, "Number of splits should match number of GEMMs."
        self.set_activation_dtype(inp)
        inp = inp.contiguous()
        # straight from the parameter table: nn.Module attribute lookup costs microseconds per name,
        # which adds up to a visible share of a step with a hundred experts
        prm = self._parameters
        weights = [prm[f"weight{i}"] for i in range(self.num_gemms)]
        biases = [prm[f"bias{i}"] for i in range(self.num_gemms)] if self.use_bias else []
        fn = _QuantizedGroupedLinear if self.qlinear_params.quantize else _NonQuantizedGroupedLinear
        grad = torch.is_grad_enabled()
        args = [] if grad else [None]
        args += [inp, m_splits, self.weight_qresult_cache, self.tp_group, self.tp_size, self.parallel_mode,
                 self.qlinear_params, self.activation_dtype, grad, is_first_microbatch, self.fuse_wgrad_accumulation,
                 *weights]
        out = (fn.apply if grad else fn.forward)(*args)
        if self.gemm_bias_unfused_add:
            shape = out.shape
            parts = torch.split(out.view(-1, self.out_features), list(m_splits))
            out = torch.cat([o + cast_if_needed(b, self.activation_dtype) for o, b in zip(parts, biases)]).view(shape)
        if self.return_bias:
            if not self.use_bias:
                biases = [getattr(self, f"bias{i}") for i in range(self.num_gemms)]
            return out, [cast_if_needed(b, self.activation_dtype) for b in biases]
        return out
