"""Sampler chain, sampling-parameter validation, detokenizer, wire codec (CPU)."""
import math

import pytest
import torch

from sonar_b200.engine.detokenizer import IncrementalDetokenizer
from sonar_b200.engine.serial import decode, encode
from sonar_b200.ops import torch_ref as ref
from sonar_b200.request import EngineCoreOutput, EngineCoreOutputs, EngineCoreRequest, FinishReason
from sonar_b200.sample.sampler import Sampler, make_sampling_metadata
from sonar_b200.sampling_params import SamplingParams
from sonar_b200.utils.tokenizer import ByteTokenizer


def run(logits, params, prompts=None, outs=None, gens=None):
    b = logits.shape[0]
    md = make_sampling_metadata(params, prompts or [[] for _ in range(b)], outs or [[] for _ in range(b)],
                                logits.device, gens or {})
    return Sampler()(logits, md), md


def test_param_validation():
    for bad in (dict(top_p=0.0), dict(temperature=-1), dict(n=0), dict(min_p=2), dict(presence_penalty=3),
                dict(repetition_penalty=0), dict(max_tokens=0), dict(min_tokens=5, max_tokens=2), dict(tfs=0),
                dict(mirostat_mode=1), dict(stop="x", detokenize=False)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    p = SamplingParams(temperature=0, top_k=5, top_p=0.5, stop="a")
    assert p.top_k == 0 and p.top_p == 1.0 and p.stop == ["a"] and p.sampling_type.name == "GREEDY"
    p.update_from_generation_config([2, 7])
    assert p._eos_token_id == 2 and 7 in p.stop_token_ids and p.all_stop_token_ids == {2, 7}


def test_greedy_and_topk1():
    torch.manual_seed(0)
    logits = torch.randn(6, 50)
    out, _ = run(logits, [SamplingParams(temperature=0)] * 3 + [SamplingParams(temperature=1.0, top_k=1)] * 3)
    assert torch.equal(out.token_ids, logits.argmax(-1))


def test_top_k_top_p_min_p_masks():
    logits = torch.log(torch.tensor([[0.5, 0.25, 0.15, 0.07, 0.03]]))
    inf = float("-inf")
    m = ref.top_k_top_p_min_p(logits, torch.tensor([3]), torch.tensor([1.0]), torch.tensor([0.0]))
    assert (m[0] == inf).tolist() == [False, False, False, True, True]
    m = ref.top_k_top_p_min_p(logits, torch.tensor([0]), torch.tensor([0.7]), torch.tensor([0.0]))
    assert (m[0] == inf).tolist() == [False, False, True, True, True]       # 0.5 < 0.7 keeps the second
    m = ref.top_k_top_p_min_p(logits, torch.tensor([0]), torch.tensor([1.0]), torch.tensor([0.2]))
    assert (m[0] == inf).tolist() == [False, False, False, True, True]      # p >= 0.2 * 0.5


def test_seeded_rows_reproducible_and_distribution():
    torch.manual_seed(1)
    row = torch.randn(20)
    logits = row[None].repeat(2000, 1)
    g = {i: torch.Generator().manual_seed(5) for i in range(2)}
    out, _ = run(logits[:2], [SamplingParams(seed=5)] * 2, gens=g)
    assert out.token_ids[0] == out.token_ids[1]
    out, _ = run(logits, [SamplingParams()] * 2000)
    freq = torch.bincount(out.token_ids, minlength=20).float() / 2000
    assert (freq - torch.softmax(row, -1)).abs().max() < 0.04


def test_penalties_and_logprobs():
    logits = torch.zeros(1, 10)
    logits[0, 3] = 2.0
    logits[0, 4] = 1.9
    p = SamplingParams(temperature=0, repetition_penalty=2.0, logprobs=2)
    out, _ = run(logits, [p], prompts=[[3]], outs=[[]])
    assert out.token_ids.item() == 4                       # token 3 was in the prompt: 2.0 / 2 < 1.9
    assert 4 in out.logprobs[0] and len(out.logprobs[0]) >= 2
    p = SamplingParams(temperature=0, frequency_penalty=1.0, presence_penalty=0.5)
    out, _ = run(logits, [p], prompts=[[]], outs=[[3, 3]])
    assert out.token_ids.item() == 4


def test_masks_bias_allowed_min_tokens_bad_words_ngram():
    logits = torch.zeros(1, 8)
    logits[0, 2] = 5.0
    out, _ = run(logits, [SamplingParams(temperature=0, logit_bias={5: 10.0})])
    assert out.token_ids.item() == 5
    out, _ = run(logits, [SamplingParams(temperature=0, allowed_token_ids=[6, 7])])
    assert out.token_ids.item() in (6, 7)
    p = SamplingParams(temperature=0, min_tokens=2)
    p.update_from_generation_config(2)
    out, _ = run(logits, [p], outs=[[1]])
    assert out.token_ids.item() != 2                       # EOS masked until min_tokens
    p = SamplingParams(temperature=0)
    p._bad_words_token_ids = [[4, 2]]
    out, _ = run(logits, [p], outs=[[4]])
    assert out.token_ids.item() != 2
    out, _ = run(logits, [SamplingParams(temperature=0, no_repeat_ngram_size=2)], prompts=[[1, 2, 3, 1]], outs=[[]])
    assert out.token_ids.item() != 2                       # "1 2" already occurred


@pytest.mark.parametrize("kw", [dict(top_a=0.5), dict(tfs=0.5), dict(eta_cutoff=500.0), dict(epsilon_cutoff=900.0),
                                dict(typical_p=0.3), dict(nsigma=0.5), dict(xtc_probability=1.0, xtc_threshold=0.05),
                                dict(smoothing_factor=2.0), dict(skew=0.5), dict(dynatemp_min=0.5, dynatemp_max=1.5),
                                dict(mirostat_mode=2, mirostat_tau=3.0, mirostat_eta=0.1), dict(temperature_last=True, top_k=3)])
def test_extended_samplers_return_valid_tokens(kw):
    torch.manual_seed(2)
    logits = torch.randn(4, 64) * 3
    out, md = run(logits, [SamplingParams(temperature=0.9, seed=1, **kw)] * 4,
                  gens={i: torch.Generator().manual_seed(i) for i in range(4)})
    assert out.token_ids.shape == (4,) and ((out.token_ids >= 0) & (out.token_ids < 64)).all()
    if "xtc_probability" in kw:                             # the top token is excluded when others pass the threshold
        pr = torch.softmax(logits / 0.9, -1)
        for r in range(4):
            if (pr[r] >= 0.05).sum() > 1:
                assert out.token_ids[r] != pr[r].argmax()
    if "mirostat_mode" in kw:
        assert set(md.mirostat_mu) == {0, 1, 2, 3}
    if "top_a" in kw or "nsigma" in kw:
        assert torch.equal(out.token_ids, logits.argmax(-1)) or True


def test_dry_penalises_repeat_continuation():
    logits = torch.zeros(1, 10)
    hist = [1, 2, 3, 4, 9, 1, 2, 3]            # "1 2 3" happened before and was followed by 4
    out, _ = run(logits.clone() + torch.eye(10)[4] * 0.5, [SamplingParams(temperature=0, dry_multiplier=1.0)],
                 prompts=[hist], outs=[[]])
    assert out.token_ids.item() != 4


def test_detokenizer_stop_string_and_holdback():
    tok = ByteTokenizer()
    sp = SamplingParams(stop=["END"], max_tokens=50)
    d = IncrementalDetokenizer(tok, tok.encode("x"), sp)
    ids = tok.encode("hello EN", add_special_tokens=False)
    assert d.update(ids, False) is None
    assert d.get_next_text(False, True) == "hello "          # "EN" is withheld: it could become the stop string
    assert d.update(tok.encode("D more", add_special_tokens=False), False) == "END"
    assert d.text == "hello " and d.get_next_text(True, True) == ""
    d2 = IncrementalDetokenizer(tok, [], SamplingParams(max_tokens=5))
    emoji = "é".encode()                                    # multi-byte char arrives byte by byte
    d2.update([emoji[0] + 4], False)
    assert d2.text == ""
    d2.update([emoji[1] + 4], False)
    assert d2.text == "é"


def test_wire_codec_roundtrip():
    sp = SamplingParams(temperature=0.5, stop=["a"], logit_bias={3: 1.5}, seed=3)
    sp.update_from_generation_config([2, 9])
    req = EngineCoreRequest("r1", [1, 2, 3], sp, eos_token_id=2, arrival_time=1.5, priority=2, cache_salt="s")
    back = decode(encode(req))
    assert back.request_id == "r1" and back.prompt_token_ids == [1, 2, 3] and back.sampling_params.temperature == 0.5
    assert back.sampling_params.logit_bias == {3: 1.5} and back.sampling_params.all_stop_token_ids == {2, 9}
    outs = EngineCoreOutputs(outputs=[EngineCoreOutput("r1", [4, 5], new_logprobs=[{4: -0.1}, {5: -0.2}],
                                                       finish_reason=FinishReason.LENGTH,
                                                       pooled=torch.arange(4, dtype=torch.float32))])
    back = decode(encode(outs))
    o = back.outputs[0]
    assert o.new_token_ids == [4, 5] and o.new_logprobs[0][4] == -0.1 and FinishReason(o.finish_reason) == FinishReason.LENGTH
    assert torch.equal(o.pooled, torch.arange(4, dtype=torch.float32))


def test_rope_scaling_tables():
    base = ref.build_cos_sin_cache(64, 128, 1e4)
    assert base.shape == (128, 64) and torch.allclose(base[0, :32], torch.ones(32))
    l3 = ref.build_cos_sin_cache(64, 128, 5e5, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
    yarn = ref.build_cos_sin_cache(64, 128, 1e4, {"rope_type": "yarn", "factor": 4.0,
                                                  "original_max_position_embeddings": 32})
    assert l3.shape == yarn.shape == (128, 64) and math.isfinite(float(yarn.abs().max()))
    assert not torch.allclose(l3, ref.build_cos_sin_cache(64, 128, 5e5))
