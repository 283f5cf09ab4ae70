"""Vocab-parallel embedding and LM head.

The vocabulary is padded to a multiple of 64·tp and split in contiguous ranges;
a lookup outside the local range yields zeros, so the sum over ranks is the
embedding.  The LM head produces the local vocab slice of the logits, which is
all-gathered along the vocab dim for the sampled rows only.

Parity: ``aphrodite/model_executor/layers/vocab_parallel_embedding.py:186,476``
and ``layers/logits_processor.py:23-96``.
"""
from __future__ import annotations

import torch
from torch import nn

from sonar_b200 import ops
from sonar_b200.parallel import state

_PAD = 64


def pad_vocab(vocab: int, tp: int) -> int:
    unit = _PAD * tp
    return -(-vocab // unit) * unit


class VocabParallelEmbedding(nn.Module):
    def __init__(self, vocab_size: int, hidden_size: int, dtype=torch.bfloat16, device=None, prefix="",
                 replicated: bool = False) -> None:
        super().__init__()
        self.tp_size, self.tp_rank = (1, 0) if replicated else (state.tp_world_size(), state.tp_rank())
        self.vocab_size = vocab_size
        self.padded = pad_vocab(vocab_size, self.tp_size)
        self.local = self.padded // self.tp_size
        self.start = self.tp_rank * self.local
        self.weight = nn.Parameter(torch.zeros(self.local, hidden_size, dtype=dtype, device=device),
                                   requires_grad=False)
        self.prefix = prefix

    def load_weight(self, name: str, tensor: torch.Tensor, shard_id=None) -> None:
        end = min(self.start + self.local, tensor.shape[0])
        if end > self.start:
            self.weight.data[: end - self.start].copy_(tensor[self.start:end])

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1:
            return torch.embedding(self.weight, input_ids.long())
        local = input_ids.long() - self.start
        ok = (local >= 0) & (local < self.local)
        out = torch.embedding(self.weight, torch.where(ok, local, torch.zeros_like(local)))
        return out * ok[:, None].to(out.dtype)


class ParallelLMHead(VocabParallelEmbedding):
    """Same storage as the embedding (and possibly the same tensor when tied)."""

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """hidden ``[B, H]`` → fp32 logits ``[B, vocab]`` on every rank."""
        local = ops.gemm(hidden, self.weight)
        if self.tp_size > 1:
            local = state.get_tp_group().all_gather(local, dim=-1)
        return local[:, : self.vocab_size].float()
