import asyncio
import json

import pytest

grpc = pytest.importorskip("grpc")

from sonar_b200.config import EngineArgs  # noqa: E402
from sonar_b200.engine.async_llm import AsyncLLM  # noqa: E402
from sonar_b200.entrypoints.grpc_server import SERVICE, create_server  # noqa: E402


def test_grpc_generate_stream_abort_health():
    args = EngineArgs(model="tiny-llama", dtype="float32", max_model_len=128, num_gpu_blocks_override=64,
                      max_num_seqs=4, max_num_batched_tokens=64, device="cpu", skip_tokenizer_init=True)
    engine = AsyncLLM.from_engine_args(args)

    def enc(o):
        return json.dumps(o).encode()

    def dec(b):
        return json.loads(b.decode())

    async def main():
        server, port = await create_server(engine, "127.0.0.1", 0)
        try:
            async with grpc.aio.insecure_channel(f"127.0.0.1:{port}") as ch:
                gen = ch.unary_stream(f"/{SERVICE}/Generate", request_serializer=enc, response_deserializer=dec)
                call = ch.unary_unary
                info = await call(f"/{SERVICE}/GetModelInfo", request_serializer=enc, response_deserializer=dec)({})
                assert info["vocab_size"] == 1024 and info["max_model_len"] == 128
                assert (await call(f"/{SERVICE}/HealthCheck", request_serializer=enc, response_deserializer=dec)({}))["healthy"]
                body = {"prompt_token_ids": [5, 6, 7, 8], "sampling_params": {"max_tokens": 6, "temperature": 0, "ignore_eos": True}}
                whole = [m async for m in gen({**body, "request_id": "a"})]
                assert len(whole) == 1 and whole[0]["finished"] and len(whole[0]["token_ids"]) == 6
                chunks = [m async for m in gen({**body, "request_id": "b", "stream": True})]
                assert sum((c["token_ids"] for c in chunks), []) == whole[0]["token_ids"] and chunks[-1]["finished"]
                assert chunks[-1]["finish_reason"] == "length" and chunks[0]["prompt_tokens"] == 4
                with pytest.raises(grpc.aio.AioRpcError) as ei:
                    [m async for m in gen({"sampling_params": {}})]
                assert ei.value.code() == grpc.StatusCode.INVALID_ARGUMENT
                with pytest.raises(grpc.aio.AioRpcError):
                    [m async for m in gen({**body, "sampling_params": {"no_such_field": 1}})]
                # abort a long request from a second call
                long_call = gen({"prompt_token_ids": [9, 9, 9], "request_id": "long", "stream": True,
                                 "sampling_params": {"max_tokens": 100, "temperature": 0, "ignore_eos": True}})
                got = []
                async for m in long_call:
                    got.append(m)
                    if len(got) == 2:
                        res = await call(f"/{SERVICE}/Abort", request_serializer=enc, response_deserializer=dec)(
                            {"request_ids": ["long", "unknown"]})
                        assert res == {"aborted": 1}
                assert got[-1]["finished"] and got[-1]["finish_reason"] == "abort" and len(got) < 100
        finally:
            await server.stop(0)
    try:
        asyncio.run(main())
    finally:
        engine.shutdown()
