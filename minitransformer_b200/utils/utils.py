"""Small helpers the linear modules use (same names as miniTransformer/utils/utils.py)."""
from typing import Callable

import torch

HIGH_PRECISION_FLOAT_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)


def is_rank_0() -> bool:
    return not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0


def init_method_normal(sigma: float) -> Callable[[torch.Tensor], torch.Tensor]:
    return lambda t: torch.nn.init.normal_(t, mean=0.0, std=sigma)


def init_method_constant(val: float) -> Callable[[torch.Tensor], torch.Tensor]:
    return lambda t: torch.nn.init.constant_(t, val)


def get_default_init_method() -> Callable[[torch.Tensor], torch.Tensor]:
    """N(0, 0.023), the reference default (miniTransformer/utils/utils.py:20-22)."""
    return init_method_normal(0.023)


def cast_if_needed(tensor, dtype: torch.dtype):
    if tensor is None or tensor.dtype == dtype:
        return tensor
    with torch.enable_grad():
        return tensor.to(dtype)


def divide(numerator: int, denominator: int) -> int:
    if numerator % denominator != 0:
        raise AssertionError(f"{numerator} is not divisible by {denominator}")
    return numerator // denominator
