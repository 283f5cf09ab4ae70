"""Analytic cost model of a decoder step: FLOPs and bytes from the architecture alone, for MFU / MBU gauges and
for roofline arithmetic in benchmarks.

* linear FLOPs per token = 2 × (parameters a token actually multiplies with): attention projections, the MLP
  or the routed + shared experts it is sent to, the LM head for sampled rows;
* attention FLOPs per token = 4 × layers × q_heads × head_dim × context (QKᵀ and PV);
* weight bytes per step = every dense weight once (+ the experts touched), KV bytes = 2 × layers × kv_heads ×
  head_dim × element size × context per decoded token.

Parity: ``aphrodite/v1/metrics/perf.py`` (per-step model FLOPs / memory traffic estimates feeding MFU metrics).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

from sonar_b200.config import ModelConfig


@dataclass
class ModelCost:
    layer_params_active: float        # weights one token multiplies with, per layer
    layer_params_total: float         # weights resident, per layer
    num_layers: int
    head_params: float                # LM head
    attn_flops_per_ctx_token: float   # per new token and per context token, all layers
    kv_bytes_per_ctx_token: float     # all layers
    weight_bytes: float               # resident weights (without embeddings)

    @classmethod
    def from_config(cls, cfg: ModelConfig, weight_elem_bytes: float | None = None, kv_elem_bytes: float = 2.0):
        g = cfg.get
        h, hd, hq, hk, n_layers = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_kv_heads, cfg.num_layers
        if cfg.is_mla:
            ql, kvl = g("q_lora_rank") or 0, g("kv_lora_rank")
            nope, rope, vd = g("qk_nope_head_dim"), g("qk_rope_head_dim"), g("v_head_dim")
            q = (h * ql + ql * hq * (nope + rope)) if ql else h * hq * (nope + rope)
            attn = q + h * (kvl + rope) + kvl * hq * (nope + vd) + hq * vd * h
            attn_flops = 4.0 * n_layers * hq * (kvl + rope)              # absorbed form works on the latent
            kv_bytes = n_layers * (kvl + rope) * kv_elem_bytes
        else:
            attn = h * (hq + 2 * hk) * hd + hq * hd * h
            attn_flops = 4.0 * n_layers * hq * hd
            kv_bytes = 2.0 * n_layers * hk * hd * kv_elem_bytes
        inter = g("intermediate_size") or 0
        n_exp = g("num_experts") or g("num_local_experts") or g("n_routed_experts") or g("moe_num_experts") or 0
        if n_exp:
            mi = g("moe_intermediate_size") or inter
            k = g("num_experts_per_tok") or g("moe_k") or 2
            shared = (g("n_shared_experts") or g("moe_num_shared_experts") or 0) * mi + (g("shared_expert_intermediate_size") or 0)
            mlp_active = 3.0 * h * (k * mi + shared) + h * n_exp
            mlp_total = 3.0 * h * (n_exp * mi + shared) + h * n_exp
        else:
            mlp_active = mlp_total = 3.0 * h * inter
        wb = weight_elem_bytes if weight_elem_bytes is not None else (1.0 if cfg.quantization else 2.0)
        head = float(h * cfg.vocab_size)
        return cls(attn + mlp_active, attn + mlp_total, n_layers, head, attn_flops, kv_bytes,
                   (n_layers * (attn + mlp_total) + head) * wb)

    def step(self, new_tokens: int, sampled_rows: int, context_tokens: float = 0.0) -> tuple[float, float]:
        """→ (FLOPs, bytes) of one step that computes ``new_tokens`` positions whose contexts sum to
        ``context_tokens`` and samples ``sampled_rows`` rows."""
        flops = 2.0 * new_tokens * self.layer_params_active * self.num_layers + 2.0 * sampled_rows * self.head_params
        flops += self.attn_flops_per_ctx_token * context_tokens
        return flops, self.weight_bytes + self.kv_bytes_per_ctx_token * context_tokens


def peaks() -> tuple[float, float]:
    """(dense bf16 FLOP/s, HBM bytes/s) the gauges are relative to: ``SONAR_PEAK_TFLOPS`` / ``SONAR_PEAK_GBS``,
    else the nominal B200 figures."""
    return float(os.environ.get("SONAR_PEAK_TFLOPS", 2250.0)) * 1e12, float(os.environ.get("SONAR_PEAK_GBS", 7700.0)) * 1e9
