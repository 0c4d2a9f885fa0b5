"""Data-parallel training on top of the fairring backend.

Two ways to use the backend for gradient all-reduce:

* ``torch.nn.parallel.DistributedDataParallel`` unchanged (the backend is a
  drop-in c10d backend), optionally with :func:`fused_allreduce_hook` so that
  the 1/W scale and a bf16/fp16 wire cast happen inside the all-reduce kernels
  instead of in separate passes over the bucket;

* :class:`FlatDataParallel`, which owns ONE flat fp32 parameter buffer and ONE
  flat gradient buffer laid out in backward order.  Gradient buckets are
  contiguous ranges of the flat gradient buffer, so a bucket is all-reduced in
  place the moment its last gradient lands -- no bucket copy-in/copy-out -- on
  the backend's side streams while backward continues, and the optimizer step
  is a single fused kernel over the flat buffers
  (:class:`fairring_b200.ops.FlatAdamW`).

The reference has no training code; what it serves is DDP's bucketed gradient
all-reduce overlapped with backward (README.md:104-110).
"""

from typing import Iterable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import get_backend


class FusedHookState:
    """State for :func:`fused_allreduce_hook`."""

    def __init__(self, process_group=None, wire_dtype: Optional[torch.dtype] = None):
        self.process_group = process_group if process_group is not None else dist.group.WORLD
        self.backend = get_backend(self.process_group, "cuda")
        self.world = dist.get_world_size(self.process_group)
        self.wire_dtype = wire_dtype


def fused_allreduce_hook(
    state: FusedHookState, bucket: dist.GradBucket
) -> torch.futures.Future[torch.Tensor]:
    """DDP communication hook: average the bucket with scale and cast fused.

    DDP does not pre-divide gradients when a hook is registered, so the kernels
    read the raw sums, multiply by 1/W while pushing, and (optionally) carry
    them as bf16/fp16 over NVLink.
    """
    buf = bucket.buffer()
    work = state.backend.allreduce_fused(buf, 1.0 / state.world, state.wire_dtype, "sum")
    return work.get_future().then(lambda f: f.value()[0])


class FlatDataParallel(nn.Module):
    """Flat-buffer data parallelism (see module docstring).

    ``bucket_cap_mb`` matches DDP's default of 25 MiB, the size the reference
    tunes its slices for (README.md:62).

    ``bf16_shadow=True`` (for training under ``torch.autocast(bfloat16)``): the
    weights and biases of ``nn.Linear`` layers are replaced by bf16 views into a
    flat shadow buffer that the optimizer kernel rewrites from the fp32 master
    weights every step.  Autocast then finds those weights already in bf16 (it
    would cast them on every forward otherwise), and their bf16 gradients are
    added into the fp32 flat gradient buffer by one small kernel each.  The
    arithmetic is what autocast does anyway -- bf16 operands, fp32 master
    weights, bf16 weight gradients widened to fp32 -- minus the cast kernels.
    Use ``FlatAdamW(ddp.flat_param, ddp.flat_grad, shadow=ddp.flat_shadow)``.
    """

    def __init__(self, module: nn.Module, process_group=None, bucket_cap_mb: float = 25.0,
                 wire_dtype: Optional[torch.dtype] = None, broadcast_parameters: bool = True,
                 symmetric_grads: bool = True, bf16_shadow: bool = False):
        super().__init__()
        self.module = module
        self.process_group = process_group if process_group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.process_group)
        self.wire_dtype = wire_dtype
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("module has no trainable parameters")
        dev = params[0].device
        if dev.type != "cuda":
            raise ValueError("FlatDataParallel needs the module on a CUDA device")
        for p in params:
            if p.dtype != torch.float32 or p.device != dev:
                raise ValueError("FlatDataParallel expects fp32 parameters on one device")
        self.device = dev
        self.backend = get_backend(self.process_group, "cuda")
        # On any other c10d backend (NCCL, say) the buckets are averaged with a
        # plain asynchronous all_reduce: same buffers, same bucket order, same
        # optimizer, only the transport differs.
        self._fused = hasattr(self.backend, "allreduce_fused")
        if not self._fused and wire_dtype is not None:
            raise ValueError("a wire dtype needs the fairring backend (fused cast)")

        # Backward produces gradients roughly in reverse registration order, so
        # lay the buffers out in that order: bucket 0 fills first.
        order = list(reversed(params))
        align = 64  # elements: keeps every parameter 256-byte aligned
        offsets, total = [], 0
        for p in order:
            offsets.append(total)
            total += (p.numel() + align - 1) // align * align
        self.flat_param = torch.zeros(total, device=dev, dtype=torch.float32)
        # Gradients live in symmetric memory when the backend offers it: every
        # rank's buffer is peer-mapped (and multicast-mapped) everywhere, so a
        # bucket is all-reduced in place by the switch, with no staging copies.
        self.symmetric = False
        if symmetric_grads and self.world > 1 and wire_dtype is None and self._fused:
            try:
                with torch.cuda.device(dev):
                    self.flat_grad = self.backend.symmetric_empty(total, torch.float32)
                self.flat_grad.zero_()
                self.symmetric = True
            except RuntimeError:
                self.symmetric = False
        if not self.symmetric:
            self.flat_grad = torch.zeros(total, device=dev, dtype=torch.float32)
        self._params = order
        self._offsets = offsets
        # name -> (offset, numel, shape) of the fp32 master copy, for state_dict()
        ids = {id(p): i for i, p in enumerate(order)}
        self._named = {n: (offsets[ids[id(p)]], p.numel(), tuple(p.shape))
                       for n, p in module.named_parameters() if id(p) in ids}
        self._index_of = dict(ids)
        self._seen = [False] * len(order)
        for p, off in zip(order, offsets):
            view = self.flat_param[off:off + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            p.grad = None

        cap = int(bucket_cap_mb * 1024 * 1024) // 4
        self._bucket_of = {}
        self._buckets = []  # [start, end) in elements
        self._bucket_size = []
        start, count = 0, 0
        for i, (p, off) in enumerate(zip(order, offsets)):
            end = offsets[i + 1] if i + 1 < len(order) else total
            self._bucket_of[id(p)] = len(self._buckets)
            count += 1
            if end - start >= cap or i + 1 == len(order):
                self._buckets.append((start, end))
                self._bucket_size.append(count)
                start, count = end, 0
        self._pending = list(self._bucket_size)
        self._next_to_launch = 0
        self._works = []
        self._callback_queued = False
        self._accumulate = False
        self._overlap_tail = False
        self._tail = None
        self.require_backward_grad_sync = True
        self._off_of = {id(p): off for p, off in zip(order, offsets)}
        for p in order:
            p.register_post_accumulate_grad_hook(self._on_grad)

        if broadcast_parameters and self.world > 1:
            dist.broadcast(self.flat_param, src=dist.get_global_rank(self.process_group, 0)
                           if self.process_group is not dist.group.WORLD else 0,
                           group=self.process_group)

        self.flat_shadow = None
        from .. import _C

        self._C = _C
        if bf16_shadow:
            self.flat_shadow = self.flat_param.to(torch.bfloat16)
            for mod in module.modules():
                if not isinstance(mod, nn.Linear):
                    continue
                for name in ("weight", "bias"):
                    master = mod._parameters.get(name)
                    if master is None or id(master) not in self._off_of:
                        continue
                    off = self._off_of[id(master)]
                    view = self.flat_shadow[off:off + master.numel()].view_as(master)
                    shadow = nn.Parameter(view, requires_grad=True)
                    mod._parameters[name] = shadow
                    self._off_of[id(shadow)] = off
                    self._bucket_of[id(shadow)] = self._bucket_of[id(master)]
                    self._index_of[id(shadow)] = self._index_of[id(master)]
                    shadow.register_post_accumulate_grad_hook(self._on_grad)

    # -- public ------------------------------------------------------------
    @property
    def num_buckets(self) -> int:
        return len(self._buckets)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def zero_grad(self, set_to_none: bool = True) -> None:  # noqa: ARG002
        """Nothing to clear here: every backward overwrites the ranges of the
        parameters that received a gradient and zeroes the ranges of those that
        did not (see ``_finish_backward``)."""
        self._accumulate = False

    def state_dict(self, *args, **kwargs) -> dict:
        """The wrapped module's state with the fp32 master weights (with
        ``bf16_shadow`` the module itself only holds bf16 copies of the
        ``nn.Linear`` parameters)."""
        sd = self.module.state_dict(*args, **kwargs)
        prefix = kwargs.get("prefix", "")
        for name, (off, n, shape) in self._named.items():
            sd[prefix + name] = self.flat_param[off:off + n].view(shape).detach().clone()
        return sd

    def load_state_dict(self, state_dict: dict, strict: bool = True):
        """Load into the fp32 master buffer (and refresh the bf16 shadow)."""
        missing = [n for n in self._named if n not in state_dict]
        if strict and missing:
            raise KeyError(f"missing parameters in state_dict: {missing[:5]}")
        with torch.no_grad():
            for name, (off, n, shape) in self._named.items():
                if name in state_dict:
                    self.flat_param[off:off + n].view(shape).copy_(state_dict[name])
            if self.flat_shadow is not None:
                self.flat_shadow.copy_(self.flat_param)
        rest = {k: v for k, v in state_dict.items() if k not in self._named}
        buffers = dict(self.module.named_buffers())
        for k, v in rest.items():
            if k in buffers:
                buffers[k].copy_(v)
            elif strict:
                raise KeyError(f"unexpected key in state_dict: {k}")

    def enable_tail_overlap(self) -> None:
        """Called by an optimizer that can start before the last bucket is
        reduced (:class:`fairring_b200.ops.FlatAdamW` with ``overlap=``): the end
        of backward then waits for every bucket but the last one, whose
        parameters (the ones whose gradients arrive last) the optimizer updates
        after waiting for it itself, see :meth:`take_tail`.  Code that reads
        ``flat_grad`` right after backward must not enable this."""
        self._overlap_tail = True

    def take_tail(self):
        """``(first element, [work, ...])`` of the bucket whose all-reduce may
        still be running, or ``None``; the caller waits for the works."""
        tail, self._tail = self._tail, None
        return tail

    def no_sync(self):
        """Context manager: accumulate locally, skip the all-reduce (like DDP's)."""
        outer = self

        class _NoSync:
            def __enter__(self_inner):
                outer.require_backward_grad_sync = False

            def __exit__(self_inner, *exc):
                outer.require_backward_grad_sync = True
                outer._accumulate = True

        return _NoSync()

    # -- backward machinery ---------------------------------------------------
    def _on_grad(self, p: torch.Tensor) -> None:
        off = self._off_of[id(p)]
        dst = self.flat_grad[off:off + p.numel()].view_as(p)
        g = p.grad
        if g.dtype == torch.bfloat16 and g.is_contiguous() and g.data_ptr() % 16 == 0:
            self._C.bf16_grad_to_f32_(dst.view(-1), g.view(-1), self._accumulate)
        elif self._accumulate:
            dst.add_(g)
        else:
            dst.copy_(g)
        p.grad = None  # the flat buffer is the gradient; views are handed out by grads()
        self._seen[self._index_of[id(p)]] = True
        if not self._callback_queued:
            torch.autograd.Variable._execution_engine.queue_callback(self._finish_backward)
            self._callback_queued = True
        b = self._bucket_of[id(p)]
        self._pending[b] -= 1
        if self.require_backward_grad_sync:
            # Launch strictly in bucket order so that every rank issues the
            # same sequence of collectives.
            while self._next_to_launch < len(self._buckets) and self._pending[self._next_to_launch] <= 0:
                self._launch(self._next_to_launch)
                self._next_to_launch += 1

    def _launch(self, b: int) -> None:
        if self.world == 1:
            return
        s, e = self._buckets[b]
        if self._fused:
            self._works.append(
                self.backend.allreduce_fused(self.flat_grad[s:e], 1.0 / self.world, self.wire_dtype, "sum")
            )
        else:
            self._works.append(
                dist.all_reduce(self.flat_grad[s:e], op=dist.ReduceOp.AVG, group=self.process_group,
                                async_op=True)
            )

    def _finish_backward(self) -> None:
        # A parameter that received no gradient in this backward must not keep
        # the (already averaged) gradient of an earlier step.
        if not self._accumulate and not all(self._seen):
            for i, seen in enumerate(self._seen):
                if not seen:
                    off = self._offsets[i]
                    self.flat_grad[off:off + self._params[i].numel()].zero_()
        self._seen = [False] * len(self._params)
        if self.require_backward_grad_sync:
            while self._next_to_launch < len(self._buckets):  # parameters that got no gradient
                self._launch(self._next_to_launch)
                self._next_to_launch += 1
            works = self._works
            self._tail = None
            if self._overlap_tail and len(works) >= 2 and len(works) == len(self._buckets):
                self._tail = (self._buckets[-1][0], [works[-1]])
                works = works[:-1]
            for w in works:
                w.wait()  # stream-level: the compute stream waits, the host does not
            self._accumulate = False
            # Host-side look at the kernels' status words (no synchronisation): a
            # device-side wait that gave up in an earlier step surfaces here, before
            # the optimizer consumes another set of gradients.
            if self._fused and self.world > 1:
                err = self.backend.health()
                if err:
                    raise RuntimeError(f"fairring: a gradient all-reduce failed ({err}); "
                                       "call backend.reset() on every rank to recover")
        else:
            self._accumulate = True
        self._works = []
        self._pending = list(self._bucket_size)
        self._next_to_launch = 0
        self._callback_queued = False

    def grads(self) -> Iterable[torch.Tensor]:
        for p, off in zip(self._params, self._offsets):
            yield self.flat_grad[off:off + p.numel()].view_as(p)
