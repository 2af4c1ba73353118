"""Output buffers of the bucketed attention operators (reference: flash3dxfmr/psh/swin_attn.py:13-43)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import plan as f3dplan


@dataclass(slots=True)
class BuckSwinFwdBuffers:
    O: torch.Tensor
    LSE: torch.Tensor

    @staticmethod
    def create_buckswin_fwd_buff(Q: torch.Tensor):
        b, l, h, _ = Q.shape
        if f3dplan.enabled():
            # inference inside plan.level_buffers(): the log-sum-exp rows are scratch nobody reads; one buffer per shape
            lse = f3dplan.pooled(("lse", b, l, h, str(Q.device)), lambda: torch.empty(b, l, h, dtype=torch.float32, device=Q.device))
            return BuckSwinFwdBuffers(torch.empty_like(Q), lse)
        return BuckSwinFwdBuffers(torch.empty_like(Q), torch.zeros(b, l, h, dtype=torch.float32, device=Q.device))


@dataclass(slots=True)
class BuckSwinBwdBuffers:
    O: torch.Tensor
    dQ: torch.Tensor
    dK: torch.Tensor
    dV: torch.Tensor
    Scope_buckets: torch.Tensor
    Delta: torch.Tensor
    buck_size: int

    @staticmethod
    def create_buckswin_buffers(O: torch.Tensor, Scope_buckets: torch.Tensor, buck_size: int):
        b, l, h, _ = O.shape
        return BuckSwinBwdBuffers(O, torch.zeros_like(O), torch.zeros_like(O), torch.zeros_like(O), Scope_buckets,
                                  torch.zeros(b, l, h, dtype=torch.float32, device=O.device), buck_size)
