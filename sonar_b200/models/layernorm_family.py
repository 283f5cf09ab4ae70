"""Decoders built on LayerNorm (with bias) and a plain GELU feed-forward: StarCoder2.

The attention, KV cache, rotary embedding and every GEMM are this package's kernels; the LayerNorm itself is
the framework's ``layer_norm`` (no kernel of its own here — these families are outside the benchmark set), so
the blocks keep the residual stream explicit instead of using the fused add+RMSNorm path, and run with
replicated activations under tensor parallelism.

Parity: ``aphrodite/model_executor/models/starcoder2.py``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from sonar_b200 import ops
from sonar_b200.config import ModelConfig
from sonar_b200.layers.linear import ColumnParallelLinear, RowParallelLinear
from sonar_b200.models.llama import LlamaAttention, LlamaForCausalLM, LlamaModel
from sonar_b200.parallel.tp_ops import get_tp_context


class LayerNorm(nn.Module):
    def __init__(self, size: int, eps: float, dtype, device) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size, dtype=dtype, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(size, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.layer_norm(x, (x.shape[-1],), self.weight, self.bias, self.eps)


class BiasedMLP(nn.Module):
    """``c_proj(act(c_fc(x)))`` with biases."""

    def __init__(self, cfg: ModelConfig, device, prefix: str) -> None:
        super().__init__()
        h, inter, bias = cfg.hidden_size, int(cfg.get("intermediate_size")), bool(cfg.get("use_bias", True))
        self.act = {"gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_new", "gelu": "gelu"}.get(
            cfg.get("hidden_act", "gelu_pytorch_tanh"), cfg.get("hidden_act"))
        self.c_fc = ColumnParallelLinear(h, [inter], bias, cfg.dtype, device, cfg.quantization, f"{prefix}.c_fc")
        self.c_proj = RowParallelLinear(inter, h, bias, cfg.dtype, device, cfg.quantization, f"{prefix}.c_proj")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tp = get_tp_context()
        return tp.row_linear(ops.activation(tp.col_linear(x, self.c_fc), self.act), self.c_proj)


class Starcoder2Attention(LlamaAttention):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__(cfg, layer_idx, device, prefix)
        if cfg.get("use_bias", True):       # q/k/v bias comes with attention_bias; the output projection has one too
            self.o_proj = RowParallelLinear(cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size, True, cfg.dtype,
                                            device, cfg.quantization, f"{prefix}.o_proj")


class Starcoder2DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__()
        eps = float(cfg.get("norm_epsilon", cfg.get("layer_norm_eps", 1e-5)))
        self.self_attn = Starcoder2Attention(cfg, layer_idx, device, f"{prefix}.self_attn")
        self.mlp = BiasedMLP(cfg, device, f"{prefix}.mlp")
        self.input_layernorm = LayerNorm(cfg.hidden_size, eps, cfg.dtype, device)
        self.post_attention_layernorm = LayerNorm(cfg.hidden_size, eps, cfg.dtype, device)

    def forward(self, h, residual, meta):
        x = h if residual is None else h + residual
        x = x + self.self_attn(self.input_layernorm(x), meta)
        x = x + self.mlp(self.post_attention_layernorm(x))
        return x, None


class Starcoder2Model(LlamaModel):
    layer_cls = Starcoder2DecoderLayer

    def __init__(self, cfg: ModelConfig, device) -> None:
        super().__init__(cfg, device)
        if self.is_last:
            self.norm = LayerNorm(cfg.hidden_size, float(cfg.get("norm_epsilon", 1e-5)), cfg.dtype, device)

    def forward(self, input_ids, meta, intermediate=None, embed_patch=None):
        tp = get_tp_context()
        if self.is_first:
            h = tp.embed_reduce(self.embed_tokens(input_ids))
            if embed_patch is not None:
                h = h.index_copy(0, embed_patch[0], embed_patch[1].to(h.dtype))
            residual = None
        else:
            h, residual = intermediate
        for layer in self.layers.values():
            h, residual = layer(h, residual, meta)
        if not self.is_last:
            return h, residual
        return self.norm(h if residual is None else h + residual)


class Starcoder2ForCausalLM(LlamaForCausalLM):
    model_cls = Starcoder2Model
    stacked_params = [(".q_proj.", ".qkv_proj.", "q"), (".k_proj.", ".qkv_proj.", "k"), (".v_proj.", ".qkv_proj.", "v")]

    def __init__(self, cfg: ModelConfig, device=None) -> None:
        cfg.hf_config.setdefault("attention_bias", bool(cfg.get("use_bias", True)))
        if cfg.get("sliding_window") and "use_sliding_window" not in cfg.hf_config:
            cfg.hf_config["use_sliding_window"] = True
        super().__init__(cfg, device)


class GPT2Model(Starcoder2Model):
    """Learned absolute positions (``wpe``) added to the token embeddings; attention layers do not rotate."""

    def __init__(self, cfg: ModelConfig, device) -> None:
        super().__init__(cfg, device)
        self.wpe = nn.Embedding(int(cfg.get("max_position_embeddings", 1024)), cfg.hidden_size, dtype=cfg.dtype, device=device)

    def forward(self, input_ids, meta, intermediate=None, embed_patch=None):
        tp = get_tp_context()
        h = tp.embed_reduce(self.embed_tokens(input_ids)) + self.wpe(meta.positions[: input_ids.shape[0]].long())
        if embed_patch is not None:
            h = h.index_copy(0, embed_patch[0], embed_patch[1].to(h.dtype))
        residual = None
        for layer in self.layers.values():
            h, residual = layer(h, residual, meta)
        return self.norm(h if residual is None else h + residual)


class GPT2LMHeadModel(Starcoder2ForCausalLM):
    """GPT-2: checkpoint tensors are ``Conv1D`` weights (``[in, out]``) with a fused ``c_attn``; they are transposed
    and cut into q / k / v when loaded."""
    model_cls = GPT2Model

    def __init__(self, cfg: ModelConfig, device=None) -> None:
        hf = cfg.hf_config
        hf.setdefault("no_rope_layers", [0] * int(hf["num_hidden_layers"]))
        hf.setdefault("tie_word_embeddings", True)
        hf.setdefault("use_bias", True)
        hf.setdefault("norm_epsilon", hf.get("layer_norm_epsilon", 1e-5))
        hf.setdefault("hidden_act", hf.get("activation_function", "gelu_new"))
        super().__init__(cfg, device)

    _RENAME = (("transformer.wte.", "model.embed_tokens."), ("transformer.wpe.", "model.wpe."), ("transformer.ln_f.", "model.norm."),
               ("transformer.h.", "model.layers."), (".ln_1.", ".input_layernorm."), (".ln_2.", ".post_attention_layernorm."),
               (".attn.c_proj.", ".self_attn.o_proj."), (".attn.c_attn.", ".self_attn.qkv_proj."))

    def load_special_weight(self, name: str, tensor: torch.Tensor) -> bool:
        from sonar_b200.loader.weights import _assign
        if name.endswith((".attn.bias", ".attn.masked_bias")):
            return True                                   # causal-mask buffers of old checkpoints
        for old, new in self._RENAME:
            name = name.replace(old, new)
        conv = any(s in name for s in (".qkv_proj.weight", ".o_proj.weight", ".c_fc.weight", ".mlp.c_proj.weight"))
        if conv:
            tensor = tensor.t()
        if ".self_attn.qkv_proj." in name:
            q, k, v = tensor.chunk(3, dim=0)
            return all([_assign(self, name, part.contiguous(), sid) for part, sid in ((q, "q"), (k, "k"), (v, "v"))])
        if name.startswith("lm_head."):
            return True
        return _assign(self, name, tensor.contiguous() if conv else tensor, None)


class NeoXDecoderLayer(Starcoder2DecoderLayer):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__(cfg, layer_idx, device, prefix)
        self.parallel = bool(cfg.get("use_parallel_residual", True))

    def forward(self, h, residual, meta):
        x = h if residual is None else h + residual
        a = self.self_attn(self.input_layernorm(x), meta)
        if self.parallel:        # both branches read the same input
            return x + a + self.mlp(self.post_attention_layernorm(x)), None
        x = x + a
        return x + self.mlp(self.post_attention_layernorm(x)), None


class NeoXModel(Starcoder2Model):
    layer_cls = NeoXDecoderLayer


class GPTNeoXForCausalLM(Starcoder2ForCausalLM):
    """GPT-NeoX / Pythia: parallel residual blocks, rotary on the first ``rotary_pct`` of each head, and a fused
    ``query_key_value`` whose rows are grouped per head as (q, k, v)."""
    model_cls = NeoXModel

    def __init__(self, cfg: ModelConfig, device=None) -> None:
        hf = cfg.hf_config
        hf.setdefault("partial_rotary_factor", hf.get("rotary_pct", 0.25))
        hf.setdefault("use_bias", bool(hf.get("attention_bias", True)))
        hf.setdefault("norm_epsilon", hf.get("layer_norm_eps", 1e-5))
        hf.setdefault("hidden_act", "gelu")
        super().__init__(cfg, device)

    _RENAME = (("gpt_neox.embed_in.", "model.embed_tokens."), ("gpt_neox.final_layer_norm.", "model.norm."),
               ("gpt_neox.layers.", "model.layers."), (".attention.dense.", ".self_attn.o_proj."),
               (".attention.query_key_value.", ".self_attn.qkv_proj."), (".mlp.dense_h_to_4h.", ".mlp.c_fc."),
               (".mlp.dense_4h_to_h.", ".mlp.c_proj."), ("embed_out.", "lm_head."))

    def load_special_weight(self, name: str, tensor: torch.Tensor) -> bool:
        from sonar_b200.loader.weights import _assign
        from sonar_b200.ops.torch_ref import partial_rotary_perm
        if "rotary_emb" in name or name.endswith((".attention.bias", ".attention.masked_bias")):
            return True
        for old, new in self._RENAME:
            name = name.replace(old, new)
        if ".self_attn.qkv_proj." not in name:
            return _assign(self, name, tensor, None)
        hd, heads = self.cfg.head_dim, self.cfg.num_attention_heads
        rot = int(hd * float(self.cfg.get("partial_rotary_factor", 1.0)))
        t = tensor.reshape(heads, 3, hd, *tensor.shape[1:])
        perm = partial_rotary_perm(hd, rot) if rot != hd else torch.arange(hd)
        parts = {"q": t[:, 0][:, perm], "k": t[:, 1][:, perm], "v": t[:, 2]}
        return all([_assign(self, name, p.reshape(heads * hd, *tensor.shape[1:]).contiguous(), sid)
                    for sid, p in parts.items()])
