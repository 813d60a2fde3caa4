"""RMSNorm part: out = x * rsqrt(mean(x^2) + eps) * (weight_offset + weight).

The reference's layer norms, per-head norms and final norm are all this operation with
the weight used as stored (pegainfer-kernels/csrc/shared/flashinfer_norm.cu:170-187); the
offset is a parameter so that a "1 + w" convention is a spec constant, not new code.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import Norm
from .registry import register_norm
from .spec import NormSpec, ParamInfo


@register_norm("rms")
class RmsNorm(Norm):
    def __init__(self, spec: NormSpec) -> None:
        super().__init__(spec)
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        return {self.spec.param_name: ParamInfo((self.spec.size,), ("one_plus_normal", 0.02))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.param_name].contiguous()

    def __call__(self, x: torch.Tensor, *, delta: Optional[torch.Tensor] = None,
                 row_idx: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        rows = x.shape[0] if row_idx is None else row_idx.numel()
        if out_dtype is not None and out_dtype != x.dtype:      # a 32-bit stream normed into the model's type
            if delta is not None:
                raise ValueError("a norm that changes the type takes no pending branch")
            out = torch.empty((rows, x.shape[1]), dtype=out_dtype, device=x.device)
            return ops.rmsnorm_cast(out, x, self.weight, self.spec.eps, row_idx=row_idx, weight_offset=self.spec.weight_offset)
        out = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
        return ops.rmsnorm(out, x, self.weight, self.spec.eps, delta=delta, row_idx=row_idx,
                           weight_offset=self.spec.weight_offset)


@register_norm("dyt")
class DynamicTanh(Norm):
    """Dynamic Tanh: out = tanh(alpha * x) * w + b with a learned scalar alpha; no mean and no variance are formed
    (``NormSpec.eps`` is not used). Tensors: the weight under ``param_name``, the bias and alpha beside it under the spec's
    suffixes. The arithmetic is float32; blocks that fuse it with the residual add take ``triple()``."""

    def __init__(self, spec: NormSpec) -> None:
        super().__init__(spec)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.alpha: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        return {s.param_name: ParamInfo((s.size,), ("one_plus_normal", 0.1)),
                s.param_name + s.bias_suffix: ParamInfo((s.size,), ("normal", 0.05)),
                s.param_name + s.alpha_suffix: ParamInfo((), ("normal_around", 0.1, 0.7))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.weight = tensors[s.param_name].contiguous()
        self.bias = tensors[s.param_name + s.bias_suffix].to(self.weight.dtype).contiguous()
        self.alpha = tensors[s.param_name + s.alpha_suffix].to(self.weight.dtype).reshape(1).contiguous()

    def triple(self):
        return self.alpha, self.weight, self.bias

    def __call__(self, x: torch.Tensor, *, delta: Optional[torch.Tensor] = None, row_idx: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if delta is not None:
            raise ValueError("a dyt norm takes no pending branch: the block that uses it joins branches itself")
        if x.dtype != torch.float32:
            raise ValueError("a dyt norm reads a float32 stream")
        rows = x.shape[0] if row_idx is None else row_idx.numel()
        out = torch.empty((rows, x.shape[1]), dtype=out_dtype or x.dtype, device=x.device)
        return ops.dyt_step(x, pre=self.triple(), out=out, row_idx=row_idx)
