"""In-place weight updates: from a checkpoint directory, and from a trainer process over the store backend;
packing helpers of the NCCL backend."""
import os
import sys
import threading

import pytest
import torch

from sonar_b200 import LLM, SamplingParams
from sonar_b200.distributed import weight_transfer as wt

sys.path.insert(0, os.path.dirname(__file__))
from tp_common import make_checkpoint  # noqa: E402

KW = dict(dtype="float32", max_model_len=128, num_gpu_blocks_override=32, device="cpu", max_num_seqs=4,
          max_num_batched_tokens=64)
SP = SamplingParams(max_tokens=8, temperature=0, ignore_eos=True)
PROMPT = [{"prompt_token_ids": list(range(30, 60))}]


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_update_from_checkpoint_directory(tmp_path):
    a = make_checkpoint(str(tmp_path / "a"), "tiny-llama-128", dtype=torch.float32, seed=0)
    b = make_checkpoint(str(tmp_path / "b"), "tiny-llama-128", dtype=torch.float32, seed=1)
    out_a = LLM(a, **KW).generate(PROMPT, SP)[0].outputs[0].token_ids
    out_b = LLM(b, **KW).generate(PROMPT, SP)[0].outputs[0].token_ids
    assert out_a != out_b
    llm = LLM(a, **KW)
    assert llm.generate(PROMPT, SP)[0].outputs[0].token_ids == out_a
    assert llm.init_weight_transfer_engine("checkpoint")
    n = llm.update_weights({"path": b})
    assert n > 10
    res = llm.generate(PROMPT, SP)[0]
    assert res.outputs[0].token_ids == out_b
    assert res.num_cached_tokens == 0                 # the old policy's prefix cache is gone
    with pytest.raises(Exception):
        llm.update_weights({"path": str(tmp_path / "missing")})


def test_update_from_trainer_over_store_backend(tmp_path):
    from sonar_b200.loader.weights import read_safetensors
    a = make_checkpoint(str(tmp_path / "a"), "tiny-llama-128", dtype=torch.float32, seed=0)
    b = make_checkpoint(str(tmp_path / "b"), "tiny-llama-128", dtype=torch.float32, seed=1)
    out_b = LLM(b, **KW).generate(PROMPT, SP)[0].outputs[0].token_ids
    new = {k: v.clone() for k, v in read_safetensors(os.path.join(b, "model.safetensors"))}
    port = _free_port()
    sender = wt.TrainerSender("store", "127.0.0.1", port, world_size=2)
    llm = LLM(a, **KW)
    t = threading.Thread(target=sender.connect)
    t.start()
    assert llm.init_weight_transfer_engine("store", sender.init_info())
    t.join(30)
    info = sender.update_info(new)
    t = threading.Thread(target=sender.send, args=(new,))
    t.start()
    assert llm.update_weights(info) == len(new)
    t.join(30)
    assert llm.generate(PROMPT, SP)[0].outputs[0].token_ids == out_b


def test_pack_plan_roundtrip_and_registry():
    tensors = {"a": torch.randn(3, 5), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(4, 4).to(torch.bfloat16),
               "d": torch.randn(100)}
    meta = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
    plan = wt.pack_plan(meta, 128)
    assert [len(g) for g in plan] == [3, 1]                # 64 + 32 + 32 bytes fill the first buffer
    for chunk in plan:
        buf = wt.pack(tensors, chunk, "cpu")
        assert buf.numel() % 16 == 0
        for name, t in wt.unpack(buf, chunk):
            assert torch.equal(t, tensors[name])
    with pytest.raises(ValueError):
        wt.create_engine("carrier-pigeon", torch.device("cpu"), 0, 1)
    assert set(wt._BACKENDS) >= {"checkpoint", "store", "nccl"}
