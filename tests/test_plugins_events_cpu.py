"""Plugin loading (in-process registration) and the KV-cache event stream with replay."""
import msgpack
import zmq

from sonar_b200 import LLM, SamplingParams
from sonar_b200 import plugins


def test_general_and_endpoint_plugins(monkeypatch):
    calls = []
    plugins.register_plugin(plugins.GENERAL, "p1", lambda: calls.append("p1"))
    plugins.register_plugin(plugins.GENERAL, "p2", lambda: calls.append("p2"))
    plugins.register_plugin(plugins.LORA_RESOLVER, "r", lambda name: f"/adapters/{name}" if name == "x" else None)
    assert set(plugins.load_general_plugins(force=True)) >= {"p1", "p2"}
    monkeypatch.setenv("SONAR_PLUGINS", "p2")
    calls.clear()
    assert plugins.load_general_plugins(force=True) == ["p2"] and calls == ["p2"]
    monkeypatch.delenv("SONAR_PLUGINS")
    assert plugins.resolve_lora("x") == "/adapters/x" and plugins.resolve_lora("y") is None


def test_kv_event_stream_and_replay():
    llm = LLM(model="tiny-llama", dtype="float32", max_model_len=128, num_gpu_blocks_override=32, device="cpu",
              max_num_seqs=4, max_num_batched_tokens=64, kv_events_endpoint="tcp://127.0.0.1:0",
              kv_events_replay_endpoint="tcp://127.0.0.1:0")
    core = llm.llm_engine.core.engine_core
    eps = core.kv_events_endpoints()
    ctx = zmq.Context.instance()
    sub = ctx.socket(zmq.SUB)
    sub.connect(eps["publish"])
    sub.setsockopt(zmq.SUBSCRIBE, b"kv-events")
    sub.setsockopt(zmq.RCVTIMEO, 200)
    llm.generate([{"prompt_token_ids": list(range(40))}], SamplingParams(max_tokens=4, temperature=0))
    # the live stream may miss the first frames (slow joiner): the replay socket has them all
    req = ctx.socket(zmq.DEALER)
    req.connect(eps["replay"])
    req.setsockopt(zmq.RCVTIMEO, 2000)
    req.send_multipart([b"", (0).to_bytes(8, "big")])
    stored = []
    while True:
        _, seq, payload = req.recv_multipart()
        if not payload:
            break
        batch = msgpack.unpackb(payload, raw=False)
        stored += [e for e in batch["events"] if e["type"] == "stored"]
    assert stored and sum(len(e["block_hashes"]) for e in stored) >= 2      # 40 prompt tokens = 2 full blocks
    assert stored[0]["token_ids"][:16] == list(range(16))
    sub.close(linger=0)
    req.close(linger=0)
    llm.shutdown()
