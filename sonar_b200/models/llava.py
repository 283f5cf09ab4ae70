"""LLaVA-1.5 family: a CLIP vision transformer, a two-layer MLP projector, and a Llama-family language model.

The language model is this package's ``LlamaForCausalLM`` (all its kernels, TP layouts and CUDA graphs apply);
the vision tower runs once per image when a request arrives — it is a few hundred tokens of dense work, done
with plain PyTorch ops, replicated on every tensor-parallel rank.  Image features come from the
``vision_feature_layer``-th hidden state (default -2: the last encoder layer is skipped), without the class
token under the default selection strategy; the projector maps them to the language model's width, and the
runner patches them over the image-token positions.

Parity: ``aphrodite/model_executor/models/llava.py`` + ``clip.py`` (feature layer selection, projector,
checkpoint names ``vision_tower.* / multi_modal_projector.* / language_model.*``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from sonar_b200.config import ModelConfig
from sonar_b200.models.llama import LlamaForCausalLM


def _act(name: str):
    if name == "quick_gelu":
        return lambda x: x * torch.sigmoid(1.702 * x)
    if name in ("gelu", "gelu_new"):
        return F.gelu
    if name in ("gelu_pytorch_tanh", "gelu_tanh"):
        return lambda x: F.gelu(x, approximate="tanh")
    raise ValueError(f"unsupported activation {name!r}")


class ClipEncoderLayer(nn.Module):
    def __init__(self, h: int, inter: int, heads: int, eps: float, act: str, dtype, device) -> None:
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.heads = heads
        self.layer_norm1, self.layer_norm2 = nn.LayerNorm(h, eps=eps, **kw), nn.LayerNorm(h, eps=eps, **kw)
        self.self_attn = nn.ModuleDict({n: nn.Linear(h, h, **kw) for n in ("q_proj", "k_proj", "v_proj", "out_proj")})
        self.mlp = nn.ModuleDict({"fc1": nn.Linear(h, inter, **kw), "fc2": nn.Linear(inter, h, **kw)})
        self.act = _act(act)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, n, h = x.shape
        y = self.layer_norm1(x)
        a = self.self_attn

        def split(t):
            return t.view(b, n, self.heads, h // self.heads).transpose(1, 2)
        o = F.scaled_dot_product_attention(split(a["q_proj"](y)), split(a["k_proj"](y)), split(a["v_proj"](y)))
        x = x + a["out_proj"](o.transpose(1, 2).reshape(b, n, h))
        return x + self.mlp["fc2"](self.act(self.mlp["fc1"](self.layer_norm2(x))))


class ClipVisionTower(nn.Module):
    """Module tree named like the checkpoint: ``vision_model.{embeddings, pre_layrnorm, encoder.layers, post_layernorm}``."""

    def __init__(self, vc: dict, dtype, device) -> None:
        super().__init__()
        h, p, size = int(vc["hidden_size"]), int(vc["patch_size"]), int(vc["image_size"])
        eps = float(vc.get("layer_norm_eps", 1e-5))
        kw = dict(dtype=dtype, device=device)
        vm = nn.Module()
        emb = nn.Module()
        emb.class_embedding = nn.Parameter(torch.zeros(h, **kw), requires_grad=False)
        emb.patch_embedding = nn.Conv2d(int(vc.get("num_channels", 3)), h, p, p, bias=False, **kw)
        emb.position_embedding = nn.Embedding((size // p) ** 2 + 1, h, **kw)
        vm.embeddings = emb
        vm.pre_layrnorm = nn.LayerNorm(h, eps=eps, **kw)          # the checkpoint's spelling
        enc = nn.Module()
        enc.layers = nn.ModuleList([
            ClipEncoderLayer(h, int(vc["intermediate_size"]), int(vc["num_attention_heads"]), eps,
                             vc.get("hidden_act", "quick_gelu"), dtype, device)
            for _ in range(int(vc["num_hidden_layers"]))])
        vm.encoder = enc
        vm.post_layernorm = nn.LayerNorm(h, eps=eps, **kw)
        self.vision_model = vm

    def forward(self, pixels: torch.Tensor, feature_layer: int) -> torch.Tensor:
        """pixels ``[B, 3, H, W]`` → hidden state number ``feature_layer`` (0 = embeddings, -1 = last layer)."""
        vm = self.vision_model
        x = vm.embeddings.patch_embedding(pixels.to(vm.embeddings.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        cls = vm.embeddings.class_embedding.expand(x.shape[0], 1, -1)
        x = torch.cat([cls, x], dim=1) + vm.embeddings.position_embedding.weight[None, : x.shape[1] + 1]
        x = vm.pre_layrnorm(x)
        n_layers = len(vm.encoder.layers)
        stop = feature_layer if feature_layer >= 0 else n_layers + 1 + feature_layer
        for layer in list(vm.encoder.layers)[:stop]:
            x = layer(x)
        return x


class LlavaForConditionalGeneration(LlamaForCausalLM):
    def __init__(self, cfg: ModelConfig, device=None) -> None:
        super().__init__(cfg, device)
        vc = cfg.get("vision_config") or {}
        if vc.get("model_type", "clip_vision_model") != "clip_vision_model":
            raise ValueError(f"vision tower {vc.get('model_type')!r} is not supported (CLIP only)")
        self.vision_tower = ClipVisionTower(vc, cfg.dtype, device)
        bias = bool(cfg.get("multimodal_projector_bias", True))
        proj = nn.Module()
        proj.linear_1 = nn.Linear(int(vc["hidden_size"]), cfg.hidden_size, bias=bias, dtype=cfg.dtype, device=device)
        proj.linear_2 = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=bias, dtype=cfg.dtype, device=device)
        self.multi_modal_projector = proj
        self.proj_act = _act(cfg.get("projector_hidden_act", "gelu"))
        layer = cfg.get("vision_feature_layer", -2)
        self.feature_layer = int(layer if not isinstance(layer, (list, tuple)) else layer[-1])
        self.drop_cls = cfg.get("vision_feature_select_strategy", "default") == "default"

    @torch.inference_mode()
    def encode_multimodal(self, kind: str, data: torch.Tensor) -> torch.Tensor:
        """Preprocessed pixel values ``[3, H, W]`` → ``[image tokens, hidden]`` rows for the placeholder positions."""
        if kind != "image":
            raise ValueError(f"unsupported modality {kind!r}")
        feats = self.vision_tower(data[None] if data.dim() == 3 else data, self.feature_layer)[0]
        if self.drop_cls:
            feats = feats[1:]
        p = self.multi_modal_projector
        return p.linear_2(self.proj_act(p.linear_1(feats)))

    def map_checkpoint_name(self, name: str):
        for old, new in (("model.language_model.model.", "model."), ("model.language_model.lm_head.", "lm_head."),
                         ("model.language_model.", "model."), ("language_model.model.", "model."),
                         ("language_model.lm_head.", "lm_head."), ("model.vision_tower.", "vision_tower."),
                         ("model.multi_modal_projector.", "multi_modal_projector.")):
            if name.startswith(old):
                name = new + name[len(old):]
                break
        if name.startswith(("vision_tower.", "multi_modal_projector.")):
            return name, None
        return super().map_checkpoint_name(name)
