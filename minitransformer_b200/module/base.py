"""Base class of the linear modules: tensor-parallel group bookkeeping, activation dtype,
deferred parameter initialisation, recipe selection. Behaviour follows
miniTransformer/module/base.py:28-191."""
import os
import warnings
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from . import config
from ..distributed.distributed import get_distributed_world_size
from ..utils.utils import get_default_init_method


@dataclass
class _ParameterInitMeta:
    init_fn: Optional[Callable] = None
    get_rng_state_tracker: Optional[Callable] = None

    def __post_init__(self):
        if self.init_fn is None:
            self.init_fn = get_default_init_method()


class LayerLinearBaseModule(torch.nn.Module, ABC):
    def __init__(self, tp_group=None, tp_size: int = 1, sequence_parallel: bool = False):
        super().__init__()
        self.tp_group_initialized = False
        if tp_group is None:
            self.tp_size = tp_size
            if tp_size == 1:
                self.set_tensor_parallel_group(None)
            # else: the caller supplies the group later through set_tensor_parallel_group()
        else:
            self.tp_size = get_distributed_world_size(tp_group)
            self.set_tensor_parallel_group(tp_group)
        self._warn_about_overlap()
        self.sequence_parallel = self.tp_size > 1 and sequence_parallel
        self.param_init_meta = {}
        self.primary_weights_in_fp8 = None
        self.fsdp_group = None

    # ---- quantized primary weights ------------------------------------------------------------
    # The reference leaves this as a placeholder (primary_weights_in_fp8 / with_fp8_params,
    # miniTransformer/module/base.py:52-58, module/linear.py:708-715). Here: once
    # keep_quantized_weights() has been called the layer's forward never re-quantizes its weight
    # (whatever is_first_microbatch says) until refresh_quantized_weights() is called, typically
    # after an optimizer step; the quantized copies travel in the state dict as extra state, so
    # a checkpoint restores them without a quantize pass.
    def keep_quantized_weights(self, keep: bool = True) -> None:
        self.primary_weights_in_fp8 = bool(keep)
        if not keep and getattr(self, "weight_qresult_cache", None) is not None:
            self.weight_qresult_cache.clear()

    def refresh_quantized_weights(self) -> None:
        """Drops the kept quantized copies; the next forward quantizes the current weights."""
        self.weight_qresult_cache.clear()

    def get_extra_state(self):
        cache = getattr(self, "weight_qresult_cache", None)
        if not self.primary_weights_in_fp8 or cache is None or cache.data is None:
            return None            # as the reference: nothing (keeps TransformerEngine checkpoints loadable)
        return {"quantized_weight": cache.state()}

    def set_extra_state(self, state: Any) -> None:
        if isinstance(state, dict) and "quantized_weight" in state:
            self.weight_qresult_cache.load_state(state["quantized_weight"])
            self.primary_weights_in_fp8 = True

    def set_activation_dtype(self, inp: torch.Tensor) -> None:
        if torch.is_autocast_enabled():
            self.activation_dtype = torch.get_autocast_gpu_dtype()
            return
        if getattr(self, "activation_dtype", None) == inp.dtype:
            return
        for name, p in self.named_parameters():
            if p is not None:
                assert inp.dtype == p.dtype, (
                    "parameter and input dtypes must match outside autocast: "
                    f"input {inp.dtype}, {name!r} {p.dtype}")
        self.activation_dtype = inp.dtype

    def set_tensor_parallel_group(self, tp_group) -> None:
        self.tp_group = tp_group
        self.tp_group_initialized = True

    def _warn_about_overlap(self) -> None:
        # Collectives overlap the backward GEMMs only if they are queued first on a single
        # hardware queue.
        if self.tp_size > 1 and int(os.getenv("CUDA_DEVICE_MAX_CONNECTIONS", "0")) != 1:
            warnings.warn("set CUDA_DEVICE_MAX_CONNECTIONS=1 to guarantee that tensor-parallel "
                          "collectives overlap the backward GEMMs")

    def register_parameter(self, name, param, **kwargs):
        super().register_parameter(name, param)
        self.param_init_meta[name] = _ParameterInitMeta(**kwargs)

    def reset_parameters(self, defer_init: Optional[bool] = False) -> None:
        if defer_init:
            return
        for name, param in self.named_parameters(recurse=False):
            if param.device == torch.device("meta"):
                param = torch.nn.Parameter(torch.empty_like(param, device="cuda"))
            meta = self.param_init_meta[name]
            if meta.get_rng_state_tracker is None:
                meta.init_fn(param)
            else:
                tracker = meta.get_rng_state_tracker()
                rng_name = getattr(self, "rng_tracker_name", None)
                with (tracker.fork(rng_name) if rng_name else tracker.fork()):
                    meta.init_fn(param)
            setattr(self, name, torch.nn.Parameter(param))

    def set_qlinear_params(self, *, qlinear_params, layer_number, layer_name):
        if qlinear_params is None:
            qlinear_params = config.get_qlinear_params_from_env_qat_params()
        if layer_number in config.get_keep_in_bf16_layer_numbers():
            return config.QLinearParams(quantize=False)
        if layer_name is not None:
            return qlinear_params.customize_for_layer_name(layer_name)
        if qlinear_params.overrides_for_layer_name:
            raise ValueError("the recipe has per-layer-name overrides but no layer name was given")
        return qlinear_params

    @abstractmethod
    def forward(self):
        ...
