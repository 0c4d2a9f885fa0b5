"""Optimizers that run as one fused kernel over flat buffers."""

from __future__ import annotations

import torch

from .. import _C


class FlatAdamW:
    """AdamW (decoupled weight decay, same update as ``torch.optim.AdamW``) over
    one flat fp32 parameter buffer and one flat fp32 gradient buffer: a single
    kernel launch per step for the whole model.

    Use with :class:`fairring_b200.parallel.FlatDataParallel`::

        ddp = FlatDataParallel(model)
        opt = FlatAdamW(ddp.flat_param, ddp.flat_grad, lr=1e-4)
    """

    def __init__(self, flat_param: torch.Tensor, flat_grad: torch.Tensor, lr: float = 1e-3,
                 betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, shadow: torch.Tensor | None = None, overlap=None):
        if flat_param.shape != flat_grad.shape or flat_param.dim() != 1:
            raise ValueError("flat_param and flat_grad must be 1-D and equally long")
        if shadow is not None and (shadow.shape != flat_param.shape or shadow.dtype != torch.bfloat16):
            raise ValueError("shadow must be a bf16 tensor as long as flat_param")
        self.param = flat_param
        self.grad = flat_grad
        self.shadow = shadow  # bf16 copy of the parameters, rewritten by every step
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.exp_avg = torch.zeros_like(flat_param)
        self.exp_avg_sq = torch.zeros_like(flat_param)
        self.step_count = 0
        # A FlatDataParallel whose last bucket may still be in flight when step()
        # is called: the parameters before it are updated first, the all-reduce
        # of the last bucket hides behind that kernel.
        self.overlap = overlap
        if overlap is not None:
            overlap.enable_tail_overlap()

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the gradient (1-element device tensor).  Waits for a
        bucket that is still being reduced."""
        tail = self.overlap.take_tail() if self.overlap is not None else None
        if tail is not None:
            for w in tail[1]:
                w.wait()
        return _C.sumsq(self.grad).sqrt()

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        tail = self.overlap.take_tail() if self.overlap is not None else None
        if tail is None:
            self._run(0, self.param.numel(), grad_scale)
            return
        off, works = tail
        self._run(0, off, grad_scale)
        for w in works:
            w.wait()
        self._run(off, self.param.numel(), grad_scale)

    def _run(self, a: int, b: int, grad_scale: float) -> None:
        if b <= a:
            return
        _C.adamw_flat_(self.param[a:b], self.grad[a:b], self.exp_avg[a:b], self.exp_avg_sq[a:b], self.lr,
                       self.betas[0], self.betas[1], self.eps, self.weight_decay,
                       self.step_count, grad_scale, None if self.shadow is None else self.shadow[a:b])

    def zero_grad(self, set_to_none: bool = True) -> None:  # noqa: ARG002
        """Gradients are overwritten by the next backward; nothing to do."""

    def state_dict(self) -> dict:
        return {"step": self.step_count, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "lr": self.lr, "betas": self.betas, "eps": self.eps,
                "weight_decay": self.weight_decay}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
