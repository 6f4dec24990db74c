"""AdamW on fp32 master weights over the flat parameter space of a ``LlamaModel``.

Single GPU: one fused kernel per step updates master/m/v, applies the global-norm clip coefficient
``min(1, clip / (norm + 1e-6))`` computed on the device, and rewrites the bf16 operational weights.

Data parallel (``DPContext`` given): each rank owns a contiguous shard of the flat space (ZeRO-1/2
style: master/m/v exist only for the shard). The step is
  barrier -> dp_reduce_norm (pull peers' fp32 grad shards over NVLink, sum, partial norm)
  -> barrier carrying the partial norms -> dp_adam_push (Adam on the shard, bf16 result stored into
  every peer's weight buffer) -> barrier.
Reference behaviour: FP32MasterAdamW and ZeRO-2 buckets (RPEG/runtime/optimizer_sharding.py:43-561,
RPEG/runtime/workers/megatron_worker.py:909-1100, 1246-1285, 3231-3338); lr 1e-6 actor / 5e-6
critic, weight decay 0, clip 1.0 are the reference defaults (RPEG/runtime/schema.py:667).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..models.llama import LlamaModel
from ..ops import kernels as K


class AdamW:
    def __init__(self, model: LlamaModel, *, lr: float = 1e-6, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, max_grad_norm: float = 1.0, dp=None, norm_group=None):
        """``norm_group``: the model is ONE PART of a larger one (a pipeline stage); the squared gradient norms of the
        parts are summed over this process group before the clip coefficient is formed, so all parts are clipped by
        the norm of the whole model."""
        if model.g is None:
            raise ValueError("optimizer needs a trainable model")
        self.model, self.lr, self.betas, self.eps, self.wd = model, lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.dp = dp
        self.norm_group = norm_group
        self.step_count = 0
        total = model.layout.total
        if dp is None or dp.world == 1:
            self.shard_off, self.shard_n = 0, total
        else:
            self.shard_off, self.shard_n = dp.shard_range(total)
        sl = slice(self.shard_off, self.shard_off + self.shard_n)
        dev = model.device
        self.master = model.w[sl].float()
        self.m = torch.zeros(self.shard_n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.shard_n, dtype=torch.float32, device=dev)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.reduced = torch.empty(self.shard_n, dtype=torch.float32, device=dev) if (dp and dp.world > 1) else None
        self.partials = torch.zeros(K.MAX_PEERS, dtype=torch.float32, device=dev)

    def state_bytes(self) -> int:
        return 12 * self.shard_n + (4 * self.shard_n if self.reduced is not None else 0)

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last ``step`` (device scalar, no sync)."""
        if self.dp is not None and self.dp.world > 1:
            return self.partials[: self.dp.world].sum().sqrt()
        return self.sumsq.sqrt()

    def step(self, grad_scale: float = 1.0, after_wait=None) -> None:
        self.step_count += 1
        m = self.model
        b1, b2 = self.betas
        if self.dp is None or self.dp.world == 1:
            self.sumsq.zero_()
            K.sumsq(m.g, self.sumsq)
            if grad_scale != 1.0:
                self.sumsq.mul_(grad_scale * grad_scale)
            if self.norm_group is not None:
                import torch.distributed as dist
                dist.all_reduce(self.sumsq, group=self.norm_group)
            K.adamw_(self.master, self.m, self.v, m.g, m.w, lr=self.lr, beta1=b1, beta2=b2, eps=self.eps, wd=self.wd,
                     step=self.step_count, grad_scale=grad_scale, sumsq=self.sumsq, max_norm=self.max_grad_norm)
            return
        self.dp.fused_adam_step(self, grad_scale, after_wait)

    # -- checkpoint helpers
    def state_dict(self) -> dict:
        return {"step": self.step_count, "shard_off": self.shard_off, "shard_n": self.shard_n,
                "master": self.master, "m": self.m, "v": self.v}

    def load_state_dict(self, sd: dict) -> None:
        if sd["shard_off"] != self.shard_off or sd["shard_n"] != self.shard_n:
            raise ValueError("optimizer shard layout differs; reshard the optimizer state first")
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
