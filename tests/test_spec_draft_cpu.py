"""Draft-model speculative decoding: the output is the target's own, whatever the draft proposes; a draft that
is the target itself gets every draft accepted; chunked prompts, prefix-cache hits and sampling are covered."""
import os
import sys

import pytest
import torch

from sonar_b200 import LLM, SamplingParams
from sonar_b200.config import EngineArgs, SpeculativeConfig

sys.path.insert(0, os.path.dirname(__file__))
from tp_common import make_checkpoint  # noqa: E402

COMMON = dict(dtype="float32", max_model_len=256, num_gpu_blocks_override=96, max_num_seqs=4,
              max_num_batched_tokens=48, device="cpu")


def _prompts():
    g = torch.Generator().manual_seed(3)
    return [{"prompt_token_ids": torch.randint(5, 120, (n,), generator=g).tolist()} for n in (9, 70, 33, 17, 50)]


def test_draft_equal_to_target_accepts_everything(tmp_path):
    ckpt = make_checkpoint(str(tmp_path / "m"), "tiny-llama-128", dtype=torch.float32)
    sp = SamplingParams(temperature=0, max_tokens=21, ignore_eos=True)
    base = LLM(ckpt, **COMMON)
    want = [o.outputs[0].token_ids for o in base.generate(_prompts(), sp)]
    base.shutdown()
    spec = LLM(ckpt, speculative_config={"model": ckpt, "num_speculative_tokens": 3}, **COMMON)
    got = [o.outputs[0].token_ids for o in spec.generate(_prompts(), sp)]
    st = spec.llm_engine.get_stats()
    assert got == want
    sched = st["scheduler"]
    assert sched.spec_num_drafts > 0 and sched.spec_num_accepted == sched.spec_num_drafts
    w = st["workers"][0]
    assert w["draft_tokens"] > 0 and w["draft_steps"] > 0
    # far fewer target steps than tokens: 21 tokens per request come out in about 21 / 4 steps
    assert w["steps"] < 5 * 21 / 2
    # a second round hits the prefix cache (the draft's KV for the cached blocks is reused too)
    again = [o.outputs[0].token_ids for o in spec.generate(_prompts(), sp)]
    assert again == want
    sched2 = spec.llm_engine.get_stats()["scheduler"]
    assert sched2.spec_num_accepted == sched2.spec_num_drafts
    spec.shutdown()


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_unrelated_draft_leaves_output_unchanged(tmp_path, temperature):
    tgt = make_checkpoint(str(tmp_path / "t"), "tiny-llama-128", dtype=torch.float32, seed=0)
    drf = make_checkpoint(str(tmp_path / "d"), "tiny-llama-128", dtype=torch.float32, seed=5)
    sps = [SamplingParams(temperature=temperature, seed=100 + i, max_tokens=12, ignore_eos=True) for i in range(5)]
    base = LLM(tgt, **COMMON)
    want = [o.outputs[0].token_ids for o in base.generate(_prompts(), sps)]
    base.shutdown()
    spec = LLM(tgt, speculative_method="draft_model", speculative_model=drf, num_speculative_tokens=2, **COMMON)
    got = [o.outputs[0].token_ids for o in spec.generate(_prompts(), sps)]
    sched = spec.llm_engine.get_stats()["scheduler"]
    spec.shutdown()
    if temperature == 0:
        assert got == want
    else:
        # rejected positions consume random numbers too, so a seeded stream is not reproduced token for token;
        # the first token (sampled before any draft exists) is, and every request runs to its length
        assert [g[0] for g in got] == [w[0] for w in want] and all(len(g) == 12 for g in got)
    assert sched.spec_num_drafts > 0 and sched.spec_num_accepted < sched.spec_num_drafts


def test_speculative_config_validation():
    assert SpeculativeConfig(model="x", num_speculative_tokens=2).method == "draft_model"
    with pytest.raises(ValueError):
        SpeculativeConfig(method="draft_model", num_speculative_tokens=2)
    with pytest.raises(ValueError):
        SpeculativeConfig(method="medusa", num_speculative_tokens=2)
    with pytest.raises(ValueError):
        SpeculativeConfig(method="ngram")
    cfg = EngineArgs(model="tiny-llama", device="cpu", dtype="float32",
                     speculative_config='{"method": "ngram", "num_speculative_tokens": 4, "prompt_lookup_max": 5}'
                     ).create_engine_config()
    assert cfg.speculative.method == "ngram" and cfg.speculative.prompt_lookup_max == 5
