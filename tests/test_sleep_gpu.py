"""Sleep mode end to end on a GPU: generate, sleep (weights offloaded, KV dropped), wake, same tokens."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_engine_sleep_wake_roundtrip():
    from sonar_b200 import LLM, SamplingParams
    llm = LLM(model="tiny-llama-128", max_model_len=256, num_gpu_blocks_override=128, max_num_seqs=8,
              max_num_batched_tokens=256, enable_sleep_mode=True, seed=0)
    sp = SamplingParams(max_tokens=8, temperature=0, ignore_eos=True)
    prompts = [{"prompt_token_ids": [3, 14, 15, 92, 65]}, {"prompt_token_ids": list(range(100, 140))}]
    before = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    freed = llm.llm_engine.sleep(1)
    free1, _ = torch.cuda.mem_get_info()
    assert freed > 0 and free1 > free0 and llm.llm_engine.is_sleeping()
    llm.llm_engine.wake_up()
    assert not llm.llm_engine.is_sleeping()
    after = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]       # CUDA graphs replay on the old addresses
    assert after == before
    llm.shutdown()
