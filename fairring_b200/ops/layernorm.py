"""LayerNorm as one kernel per direction (``csrc/kernels/layernorm.cu``).

Under ``torch.autocast(bfloat16)`` torch computes layer_norm in fp32 and the
linear layer behind it casts the result to bf16 in a pass of its own; the
backward is two more kernels.  :class:`FusedLayerNorm` reads the row once,
writes the output directly in the autocast dtype and keeps two floats per row
for the backward, which reads ``dy`` and ``x`` once and reduces the weight and
bias gradients on the way.  Same parameters and state dict as
``torch.nn.LayerNorm``; falls back to it off the GPU, for dtypes other than
fp32/bf16 and for row lengths that are not a multiple of 8 or exceed 8192.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import _C


class _FusedLayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_dtype):
        xc = x.contiguous()
        y, mean, rstd = _C.layer_norm_fwd(xc, weight, bias, eps, out_dtype)
        ctx.save_for_backward(xc, weight, mean, rstd)
        ctx.out_dtype = out_dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, mean, rstd = ctx.saved_tensors
        if dy.dtype != ctx.out_dtype:
            dy = dy.to(ctx.out_dtype)
        dx, dgamma, dbeta = _C.layer_norm_bwd(dy.contiguous(), x, weight, mean, rstd)
        return dx, dgamma, dbeta, None, None


def fused_layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5,
                     out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """LayerNorm over the last dimension; ``out_dtype`` defaults to the autocast
    dtype inside an autocast region and to ``x.dtype`` otherwise."""
    if out_dtype is None:
        out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
    return _FusedLayerNormFn.apply(x, weight, bias, eps, out_dtype)


class FusedLayerNorm(nn.LayerNorm):
    def _fusable(self, x: torch.Tensor) -> bool:
        d = x.shape[-1]
        return (x.is_cuda and len(self.normalized_shape) == 1 and self.weight is not None
                and self.bias is not None and self.weight.dtype == torch.float32
                and x.dtype in (torch.float32, torch.bfloat16) and d % 8 == 0 and d <= 8192)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self._fusable(x):
            return super().forward(x)
        out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        if out_dtype not in (torch.float32, torch.bfloat16):
            return super().forward(x)
        return _FusedLayerNormFn.apply(x, self.weight, self.bias, self.eps, out_dtype)


class _AddLayerNormFn(torch.autograd.Function):
    """(x + branch, LayerNorm(x + branch)) in one kernel; the backward adds the
    gradient that reaches the sum along the residual path inside the LayerNorm
    backward kernel and hands the result to both addends."""

    @staticmethod
    def forward(ctx, x, branch, weight, bias, eps, out_dtype):
        xnew, y, mean, rstd = _C.add_layer_norm_fwd(x.contiguous(), branch.contiguous(), weight, bias, eps,
                                                    out_dtype)
        ctx.save_for_backward(xnew, weight, mean, rstd)
        ctx.set_materialize_grads(False)  # an unused output arrives as None, not as zeros
        ctx.out_dtype = out_dtype
        ctx.branch_dtype = branch.dtype
        return xnew, y

    @staticmethod
    def backward(ctx, g_xnew, dy):
        xnew, weight, mean, rstd = ctx.saved_tensors
        if dy is None:  # the normalised output was not used: only the residual path carries gradient
            g = g_xnew if g_xnew is not None else torch.zeros_like(xnew)
            return g, g.to(ctx.branch_dtype), torch.zeros_like(weight), torch.zeros_like(weight), None, None
        if dy.dtype != ctx.out_dtype:
            dy = dy.to(ctx.out_dtype)
        gres = None if g_xnew is None else g_xnew.float().contiguous()
        want_bf16 = ctx.branch_dtype == torch.bfloat16
        dx, dbr, dgamma, dbeta = _C.add_layer_norm_bwd(dy.contiguous(), xnew, weight, mean, rstd, gres, want_bf16)
        return dx, (dbr if want_bf16 else dx), dgamma, dbeta, None, None


def add_layer_norm(norm: nn.LayerNorm, x: torch.Tensor, branch: torch.Tensor | None):
    """``(x + branch, norm(x + branch))``.  One kernel each way when ``norm`` is a
    :class:`FusedLayerNorm`, ``x`` is the fp32 residual stream on the GPU and
    ``branch`` is fp32 or bf16; plain torch otherwise.  ``branch=None`` skips the add."""
    if branch is None:
        return x, norm(x)
    fusable = (isinstance(norm, FusedLayerNorm) and norm._fusable(x) and x.dtype == torch.float32
               and branch.dtype in (torch.float32, torch.bfloat16) and branch.shape == x.shape
               and branch.device == x.device)
    if fusable:
        out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        if out_dtype in (torch.float32, torch.bfloat16):
            return _AddLayerNormFn.apply(x, branch, norm.weight, norm.bias, norm.eps, out_dtype)
    xnew = x + branch
    return xnew, norm(xnew)
