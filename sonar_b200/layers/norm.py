"""RMSNorm module (weights only; math in ``sonar_b200.ops``).
Parity: ``aphrodite/model_executor/layers/layernorm.py:35``."""
from __future__ import annotations

import torch
from torch import nn

from sonar_b200 import ops


class RMSNorm(nn.Module):
    def __init__(self, size: int, eps: float = 1e-6, dtype=torch.bfloat16, device=None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps

    def load_weight(self, name: str, tensor: torch.Tensor, shard_id=None) -> None:
        self.weight.data.copy_(tensor)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if residual is None:
            return ops.rms_norm(x, self.weight, self.eps)
        return ops.fused_add_rms_norm(x, residual, self.weight, self.eps)
