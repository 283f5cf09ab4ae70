"""Prompts given as embeddings: feeding the embedding-table rows of a token prompt reproduces that prompt's
output, also when the prompt is prefilled in chunks and mixed with ordinary requests."""
import pytest
import torch

from sonar_b200 import LLM, SamplingParams


def test_prompt_embeds_match_token_prompt():
    kw = dict(model="tiny-llama", dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks_override=48,
              max_num_seqs=4, max_num_batched_tokens=16, seed=0)          # 16-token budget: chunked prefill
    sp = SamplingParams(temperature=0, max_tokens=6, ignore_eos=True)
    ids_a, ids_b = list(range(30, 70)), list(range(200, 223))
    llm = LLM(**kw)
    want = [o.outputs[0].token_ids for o in llm.generate([{"prompt_token_ids": ids_a}, {"prompt_token_ids": ids_b}], sp)]
    table = llm.llm_engine.core.engine_core.executor.worker.runner.model.model.embed_tokens.weight
    emb_a = table[torch.tensor(ids_a)].clone()
    llm.reset_prefix_cache()
    outs = llm.generate([{"prompt_embeds": emb_a}, {"prompt_token_ids": ids_b}], sp)
    assert [o.outputs[0].token_ids for o in outs] == want
    assert len(outs[0].prompt_token_ids) == len(ids_a)
    # other embeddings, same placeholder ids: no false prefix-cache hit, different continuation
    other = llm.generate([{"prompt_embeds": emb_a.flip(0)}], sp)[0]
    assert other.num_cached_tokens == 0
    # the same embeddings again do hit the cache
    again = llm.generate([{"prompt_embeds": emb_a}], sp)[0]
    assert again.outputs[0].token_ids == want[0] and again.num_cached_tokens >= 32
    with pytest.raises(ValueError):
        llm.generate([{"prompt_embeds": torch.zeros(4, 7)}], sp)
    llm.shutdown()
