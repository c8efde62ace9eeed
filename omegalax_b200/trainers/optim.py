"""Mixed-precision AdamW: fp32 master weights and moments, bf16 compute copies.

``MixedPrecisionOptimizer`` is the sharded train engine with the optimizer-facing surface
the trainers use (model, step counter, update).  Gradients are accumulated in fp32, the
update is ``p <- p - lr * (m_hat / (sqrt(v_hat) + eps) + wd * p)`` on the fp32 master and the
compute copy is the rounded master (reference: omegalax/trainers/optim.py:11-41; AdamW with
beta=(0.9, 0.999), eps=1e-8, decay applied to every parameter, optional global-norm clip and
k-step gradient accumulation as in omegalax/trainers/text.py:71-88).
"""
from __future__ import annotations

from ..parallel.engine import TrainEngine


class MixedPrecisionOptimizer(TrainEngine):
    def __init__(self, model, *, lr_schedule=None, grad_accum_steps: int = 1, **kw):
        super().__init__(model, **kw)
        self.lr_schedule = lr_schedule
        self.grad_accum_steps = max(int(grad_accum_steps), 1)
        self.last_grad_norm = None

    @property
    def step(self) -> int:
        return self.step_count

    def update(self):
        """Call after every micro-batch backward.  Applies the optimizer every
        ``grad_accum_steps`` calls; returns the pre-clip gradient norm when it did."""
        self.finish_backward()
        if self.micro_steps < self.grad_accum_steps:
            return None
        lr = self.lr_schedule(self.step_count) if self.lr_schedule is not None else self.lr
        self.last_grad_norm = self.optimizer_step(lr=lr, grad_accum=self.grad_accum_steps)
        return self.last_grad_norm
