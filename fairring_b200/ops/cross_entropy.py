"""Softmax cross-entropy for language-model heads in two kernels
(``csrc/kernels/cross_entropy.cu``): the forward keeps one float per row, the
backward writes the gradient over the logits in their own dtype.  The logits
must not be used after the loss (their memory becomes their gradient) -- true
for a language-model head, where the loss is their only consumer.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _C


class _FusedCrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        losses, lse = _C.cross_entropy_fwd(logits, targets)
        valid = (targets >= 0).sum().clamp_(min=1)
        ctx.save_for_backward(logits, targets, lse, valid)
        return losses.sum() / valid

    @staticmethod
    def backward(ctx, g):
        logits, targets, lse, valid = ctx.saved_tensors
        upstream = (g.float() / valid).reshape(1)
        grad = logits.detach()
        _C.cross_entropy_bwd_(grad, targets, lse, upstream, 1.0)
        return grad, None


def fused_cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy of ``logits`` [rows, vocab] (fp32 or bf16) against
    ``targets`` [rows] (negative entries are ignored).  Consumes the logits: after
    backward their storage holds the gradient.  Falls back to
    ``F.cross_entropy(logits.float(), targets)`` off the GPU and for shapes the
    kernels do not take."""
    ok = (logits.is_cuda and logits.dim() == 2 and logits.is_contiguous()
          and logits.dtype in (torch.float32, torch.bfloat16) and logits.shape[1] % 8 == 0
          and targets.dtype == torch.long)
    if not ok:
        return F.cross_entropy(logits.float(), targets, ignore_index=-100)
    return _FusedCrossEntropyFn.apply(logits, targets.contiguous())
