"""LoRA adapters: a PEFT-format adapter applied through the slot kernels equals the merged-weight model."""
import json
import os

import pytest
import torch

from sonar_b200 import LLM, SamplingParams
from sonar_b200.loader.weights import write_safetensors
from sonar_b200.lora import LoRARequest


def _make_adapter(path, cfg, r=8, alpha=16.0, seed=0, modules=("q_proj", "v_proj", "gate_proj", "down_proj")):
    g = torch.Generator().manual_seed(seed)
    h, inter = cfg["hidden_size"], cfg["intermediate_size"]
    hd = cfg["head_dim"]
    dims = {"q_proj": (cfg["num_attention_heads"] * hd, h), "k_proj": (cfg["num_key_value_heads"] * hd, h),
            "v_proj": (cfg["num_key_value_heads"] * hd, h), "o_proj": (h, cfg["num_attention_heads"] * hd),
            "gate_proj": (inter, h), "up_proj": (inter, h), "down_proj": (h, inter)}
    tensors = {}
    for layer in range(cfg["num_hidden_layers"]):
        for m in modules:
            n, k = dims[m]
            parent = "self_attn" if m in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            base = f"base_model.model.model.layers.{layer}.{parent}.{m}"
            tensors[f"{base}.lora_A.weight"] = torch.randn(r, k, generator=g) * 0.3
            tensors[f"{base}.lora_B.weight"] = torch.randn(n, r, generator=g) * 0.3
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "adapter_model.safetensors"), tensors)
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": alpha, "target_modules": list(modules), "peft_type": "LORA"}, f)
    return tensors, alpha / r


def test_lora_matches_merged_weights_and_mixes_adapters_in_one_batch(tmp_path):
    from sonar_b200.config import ARCH_PRESETS
    cfg = ARCH_PRESETS["tiny-llama"]
    a1 = str(tmp_path / "a1")
    a2 = str(tmp_path / "a2")
    t1, sc1 = _make_adapter(a1, cfg, seed=1)
    _make_adapter(a2, cfg, seed=2, modules=("k_proj", "o_proj", "up_proj"))
    kw = dict(model="tiny-llama", dtype="float32", max_model_len=128, num_gpu_blocks_override=64, device="cpu",
              max_num_seqs=8, max_num_batched_tokens=64, seed=0)
    sp = SamplingParams(max_tokens=8, temperature=0, ignore_eos=True)
    prompts = [{"prompt_token_ids": [5, 6, 7, 8, 9]}, {"prompt_token_ids": [100, 90, 80]}]

    llm = LLM(**kw, enable_lora=True, max_loras=2, max_lora_rank=8)
    base = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    with_a1 = [o.outputs[0].token_ids for o in llm.generate(prompts, sp, lora_request=LoRARequest("a1", 1, a1))]
    # one batch: prompt 0 with adapter a1, prompt 1 with a2, plus a plain one
    mixed = llm.generate(prompts + [prompts[0]], sp,
                         lora_request=[LoRARequest("a1", 1, a1), LoRARequest("a2", 2, a2), None])
    assert mixed[0].outputs[0].token_ids == with_a1[0]
    assert mixed[2].outputs[0].token_ids == base[0]
    assert with_a1 != base
    assert llm.llm_engine.list_loras() == ["a1", "a2"]
    # unknown adapter
    with pytest.raises(Exception):
        llm.generate(prompts[:1], sp, lora_request=LoRARequest("nope", 9, str(tmp_path / "missing")))

    # reference: merge a1 into the base weights of a fresh engine
    ref = LLM(**kw)
    model = ref.llm_engine.core.engine_core.executor.worker.runner.model
    for name, t in t1.items():
        if ".lora_A." not in name:
            continue
        mod = name[len("base_model.model."):].split(".lora_A")[0]
        a, b = t, t1[name.replace("lora_A", "lora_B")]
        delta = (b @ a) * sc1
        parent, leaf = mod.rsplit(".", 1)
        attr, sub = {"q_proj": ("qkv_proj", 0), "v_proj": ("qkv_proj", 2), "gate_proj": ("gate_up_proj", 0),
                     "down_proj": ("down_proj", 0)}[leaf]
        layer = model.get_submodule(f"{parent}.{attr}")
        off = sum(layer.local_sizes[:sub]) if hasattr(layer, "local_sizes") else 0
        with torch.inference_mode():
            layer.weight.data[off:off + delta.shape[0]] += delta
    merged = [o.outputs[0].token_ids for o in ref.generate(prompts, sp)]
    assert merged == with_a1
    assert llm.llm_engine.remove_lora("a2") and llm.llm_engine.list_loras() == ["a1"]
