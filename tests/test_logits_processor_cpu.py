import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(__file__))

from sonar_b200 import LLM, SamplingParams  # noqa: E402
from sonar_b200.config import EngineArgs  # noqa: E402

KW = dict(model="tiny-llama", dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks_override=32,
          max_num_seqs=4, max_num_batched_tokens=64)


def test_custom_processors_by_name_and_class():
    import lp_fixtures
    llm = LLM(**KW, logits_processors=["lp_fixtures:ForceToken", lp_fixtures.NoImmediateRepeat], async_scheduling=True)
    core = llm.llm_engine.core.engine_core
    assert not core.run_ahead_ok                                   # lock-step while custom processors exist
    prompts = [{"prompt_token_ids": [5, 6, 7, 8]}, {"prompt_token_ids": [9, 10, 11]}, {"prompt_token_ids": [3, 4]}]
    sps = [SamplingParams(max_tokens=4, temperature=0, ignore_eos=True, extra_args={"force_token": 42}),
           SamplingParams(max_tokens=12, temperature=0, ignore_eos=True),
           SamplingParams(max_tokens=6, temperature=0.8, seed=1, ignore_eos=True)]
    outs = llm.generate(prompts, sps)
    # processors run in the order given: the first leaves token 42 as the only finite logit; from the second
    # step on the other processor bans the previous token as well, so only the first token is pinned down
    assert outs[0].outputs[0].token_ids[0] == 42
    for o in outs[1:]:
        t = o.outputs[0].token_ids
        assert all(a != b for a, b in zip(t, t[1:]))               # never the same token twice in a row
    assert lp_fixtures.ForceToken.calls >= 1
    llm.shutdown()


def test_bad_names_are_rejected_and_cli_parses_a_json_list():
    import argparse
    with pytest.raises((ImportError, AttributeError, TypeError)):
        LLM(**KW, logits_processors=["lp_fixtures:Missing"])
    with pytest.raises(TypeError):
        LLM(**KW, logits_processors=["os.path:join"])
    ns = EngineArgs.add_cli_args(argparse.ArgumentParser()).parse_args(["--logits-processors", '["lp_fixtures:ForceToken"]'])
    assert EngineArgs.from_cli_args(ns).logits_processors == ["lp_fixtures:ForceToken"]
