"""AWQ / GPTQ checkpoints: packing layouts, dequantisation, and an engine that loads them and reproduces the
output of the same (quantised-then-widened) weights stored as plain tensors."""
import json
import os
import sys

import pytest
import torch

from sonar_b200 import LLM, SamplingParams
from sonar_b200.loader import int4
from sonar_b200.loader.weights import read_safetensors, save_checkpoint

sys.path.insert(0, os.path.dirname(__file__))
from tp_common import make_checkpoint  # noqa: E402


def _quantize(w: torch.Tensor, group: int, sym: bool):
    """[out, in] → nibbles [in, out], zeros [in/g, out], scales [in/g, out] (asymmetric min/max per group)."""
    wt = w.t().float()
    n_in, n_out = wt.shape
    g = wt.reshape(n_in // group, group, n_out)
    if sym:
        s = g.abs().amax(1) / 7
        z = torch.full_like(s, 8)
    else:
        lo, hi = g.amin(1), g.amax(1)
        s = (hi - lo).clamp(min=1e-6) / 15
        z = (-lo / s).round().clamp(0, 15)
    s = s.to(torch.float16)
    q = (g / s.float()[:, None] + z[:, None]).round().clamp(0, 15).reshape(n_in, n_out)
    return q.to(torch.int32), z.to(torch.int32), s


def test_unpackers_invert_packers():
    torch.manual_seed(0)
    q = torch.randint(0, 16, (32, 64), dtype=torch.int32)
    assert torch.equal(int4._unpack_cols(int4.pack_cols(q)), q)
    assert torch.equal(int4._unpack_rows(int4.pack_rows(q)), q)
    # AWQ order: nibble i of a word holds column order[i] of its group of eight
    word = int4.pack_awq(torch.arange(8, dtype=torch.int32)[None])
    assert [(int(word[0, 0]) >> (4 * i)) & 15 for i in range(8)] == [0, 2, 4, 6, 1, 3, 5, 7]


@pytest.mark.parametrize("method,sym", [("awq", False), ("gptq", False), ("gptq", True)])
def test_dequantisation_formulas(method, sym):
    torch.manual_seed(1)
    w = torch.randn(48, 64) * 0.1
    q, z, s = _quantize(w, 32, sym)
    want = ((q - z.repeat_interleave(32, 0)).float() * s.float().repeat_interleave(32, 0)).t()
    if method == "awq":
        got = int4.dequantize_awq(int4.pack_awq(q), int4.pack_awq(z), s, 32)
    else:
        g_idx = torch.arange(64) // 32
        got = int4.dequantize_gptq(int4.pack_rows(q), int4.pack_cols(z - 1), s, 32, g_idx)
    assert got.shape == (48, 64) and torch.allclose(got.float(), want, atol=1e-3)
    assert (got.float() - w).abs().max() < 0.05                   # and it is a 4-bit approximation of w


@pytest.mark.parametrize("method", ["awq", "gptq"])
def test_engine_loads_int4_checkpoint(tmp_path, method):
    base = make_checkpoint(str(tmp_path / "base"), "tiny-llama-128", dtype=torch.float32)
    cfg = json.load(open(os.path.join(base, "config.json")))
    tensors = dict(read_safetensors(os.path.join(base, "model.safetensors")))
    packed, widened = {}, {}
    for name, t in tensors.items():
        if name.endswith("_proj.weight"):
            q, z, s = _quantize(t, 32, False)
            pre = name[: -len(".weight")]
            if method == "awq":
                packed[pre + ".qweight"], packed[pre + ".qzeros"] = int4.pack_awq(q), int4.pack_awq(z)
            else:
                packed[pre + ".qweight"], packed[pre + ".qzeros"] = int4.pack_rows(q), int4.pack_cols(z - 1)
                packed[pre + ".g_idx"] = (torch.arange(q.shape[0]) // 32).int()
            packed[pre + ".scales"] = s
            widened[name] = ((q - z.repeat_interleave(32, 0)).float() * s.float().repeat_interleave(32, 0)).t().contiguous()
        else:
            packed[name] = widened[name] = t.clone()
    qcfg = {"quant_method": method, "bits": 4, "group_size": 32, "zero_point": True, "version": "gemm", "desc_act": False}
    save_checkpoint(str(tmp_path / "q"), {**cfg, "quantization_config": qcfg}, packed)
    save_checkpoint(str(tmp_path / "w"), cfg, widened)
    kw = dict(dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks_override=32, max_num_seqs=2,
              max_num_batched_tokens=64, skip_tokenizer_init=True)
    sp = SamplingParams(temperature=0, max_tokens=8, logprobs=1, ignore_eos=True, detokenize=False)
    prompt = [{"prompt_token_ids": list(range(40, 70))}]
    want = LLM(str(tmp_path / "w"), **kw).generate(prompt, sp)[0].outputs[0]
    llm = LLM(str(tmp_path / "q"), **kw)
    assert llm.llm_engine.cfg.model.int4_config["quant_method"] == method
    got = llm.generate(prompt, sp)[0].outputs[0]
    assert list(got.token_ids) == list(want.token_ids)
    plain = LLM(base, **kw).generate(prompt, sp)[0].outputs[0]
    assert len(plain.token_ids) == 8                                # the unquantised model runs too (sanity)


@pytest.mark.parametrize("sym", [True, False])
def test_compressed_tensors_pack_quantized(tmp_path, sym):
    torch.manual_seed(2)
    w = torch.randn(40, 64) * 0.1
    q, z, s = _quantize(w, 32, sym)                                # q [in, out], z/s [in/g, out]
    want = ((q - z.repeat_interleave(32, 0)).float() * s.float().repeat_interleave(32, 0)).t()
    packed = int4.pack_cols(q.t().contiguous())                   # [out, in/8]
    zp = None if sym else int4.pack_rows(z.t().contiguous())      # [out/8, in/g]
    got = int4.dequantize_compressed_tensors(packed, s.t().contiguous(), zp, 32, (40, 64))
    assert torch.allclose(got.float(), want, atol=1e-3)
    qcfg = {"quant_method": "compressed-tensors", "format": "pack-quantized",
            "config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": 32, "symmetric": sym}}}}
    stream = [("a.norm.weight", torch.ones(4)), ("a.proj.weight_packed", packed), ("a.proj.weight_scale", s.t().contiguous()),
              ("a.proj.weight_shape", torch.tensor([40, 64]))]
    if not sym:
        stream.append(("a.proj.weight_zero_point", zp))
    out = dict(int4.widen_int4_checkpoint(iter(stream), qcfg))
    assert set(out) == {"a.norm.weight", "a.proj.weight"} and torch.allclose(out["a.proj.weight"].float(), want, atol=1e-3)
