"""gRPC front end of the engine (token-in / token-out, for routers that keep tokenisation to themselves).

Service ``sonar.Engine`` with JSON-encoded messages over generic method handlers (no generated stubs, so no
``protoc`` step):

* ``Generate``      unary → stream: ``{"request_id", "prompt_token_ids" | "prompt", "sampling_params": {…},
  "stream": bool}`` → chunks ``{"request_id", "token_ids", "text", "finished", "finish_reason",
  "prompt_tokens", "cached_tokens"}`` (deltas when ``stream``; one final message otherwise);
* ``Abort``         ``{"request_ids": […]}`` → ``{"aborted": n}``;
* ``HealthCheck``   ``{}`` → ``{"healthy": bool}``;
* ``GetModelInfo``  ``{}`` → model name, vocabulary size, context length, parallel sizes.

``python -m sonar_b200.entrypoints.grpc_server --model … --port 50051`` starts it.

Parity: ``aphrodite/entrypoints/grpc_server.py`` (an ``AsyncLLM``-backed servicer with Generate / Abort /
HealthCheck / GetModelInfo, unlimited message sizes, keep-alive options); that file takes its message types
from an external package, so the wire format here is this build's own.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import uuid
from typing import Any

from sonar_b200.logger import init_logger
from sonar_b200.sampling_params import SamplingParams

logger = init_logger(__name__)
SERVICE = "sonar.Engine"


def _dumps(obj: Any) -> bytes:
    return json.dumps(obj).encode()


def _loads(raw: bytes) -> Any:
    return json.loads(raw.decode() or "{}")


class EngineServicer:
    def __init__(self, engine) -> None:
        self.engine = engine
        self.active: set[str] = set()

    async def generate(self, req: dict, context):
        import grpc
        rid = req.get("request_id") or f"grpc-{uuid.uuid4().hex}"
        prompt = req.get("prompt")
        if req.get("prompt_token_ids") is not None:
            prompt = {"prompt_token_ids": list(req["prompt_token_ids"])}
        if prompt is None:
            await context.abort(grpc.StatusCode.INVALID_ARGUMENT, "prompt or prompt_token_ids is required")
        try:
            sp = SamplingParams(**(req.get("sampling_params") or {}))
            gen = self.engine.generate(prompt, sp, rid, priority=int(req.get("priority", 0)))
        except (TypeError, ValueError) as e:
            await context.abort(grpc.StatusCode.INVALID_ARGUMENT, str(e))
        stream = bool(req.get("stream", False))
        sent = 0
        self.active.add(rid)
        try:
            final = None
            async for out in gen:
                final = out
                c = out.outputs[0]
                if stream:
                    ids = list(c.token_ids)
                    yield {"request_id": rid, "token_ids": ids[sent:], "text": c.text, "finished": out.finished,
                           "finish_reason": c.finish_reason, "prompt_tokens": len(out.prompt_token_ids or []),
                           "cached_tokens": out.num_cached_tokens}
                    sent = len(ids)
            if not stream and final is not None:
                c = final.outputs[0]
                yield {"request_id": rid, "token_ids": list(c.token_ids), "text": c.text, "finished": True,
                       "finish_reason": c.finish_reason, "prompt_tokens": len(final.prompt_token_ids or []),
                       "cached_tokens": final.num_cached_tokens}
        except asyncio.CancelledError:
            await self.engine.abort(rid)          # the client went away
            raise
        finally:
            self.active.discard(rid)

    async def abort(self, req: dict, context) -> dict:
        ids = [r for r in req.get("request_ids", []) if r in self.active]
        for r in ids:
            await self.engine.abort(r)
        return {"aborted": len(ids)}

    async def health(self, req: dict, context) -> dict:
        return {"healthy": bool(self.engine.is_running)}

    async def model_info(self, req: dict, context) -> dict:
        cfg = self.engine.cfg
        return {"model": cfg.model.served_model_name, "vocab_size": cfg.model.vocab_size,
                "max_model_len": cfg.model.max_model_len, "tensor_parallel_size": cfg.parallel.tensor_parallel_size,
                "data_parallel_size": cfg.parallel.data_parallel_size}


def add_servicer(server, servicer: EngineServicer) -> None:
    import grpc
    handlers = {
        "Generate": grpc.unary_stream_rpc_method_handler(servicer.generate, _loads, _dumps),
        "Abort": grpc.unary_unary_rpc_method_handler(servicer.abort, _loads, _dumps),
        "HealthCheck": grpc.unary_unary_rpc_method_handler(servicer.health, _loads, _dumps),
        "GetModelInfo": grpc.unary_unary_rpc_method_handler(servicer.model_info, _loads, _dumps),
    }
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(SERVICE, handlers),))


async def create_server(engine, host: str = "127.0.0.1", port: int = 50051):
    """→ (started ``grpc.aio`` server, bound port)."""
    import grpc
    server = grpc.aio.server(options=[("grpc.max_send_message_length", -1), ("grpc.max_receive_message_length", -1),
                                      ("grpc.keepalive_permit_without_calls", True),
                                      ("grpc.http2.min_recv_ping_interval_without_data_ms", 10000)])
    add_servicer(server, EngineServicer(engine))
    bound = server.add_insecure_port(f"{host}:{port}")
    await server.start()
    return server, bound


def main(argv: list[str] | None = None) -> None:
    from sonar_b200.config import EngineArgs
    from sonar_b200.engine.async_llm import AsyncLLM
    ap = argparse.ArgumentParser(prog="sonar-grpc")
    ap.add_argument("--model", required=True)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=50051)
    EngineArgs.add_cli_args(ap)
    ns = ap.parse_args(argv)
    engine = AsyncLLM.from_engine_args(EngineArgs.from_cli_args(ns))

    async def run() -> None:
        server, port = await create_server(engine, ns.host, ns.port)
        logger.info("gRPC server on %s:%d (service %s)", ns.host, port, SERVICE)
        try:
            await server.wait_for_termination()
        finally:
            await server.stop(2)
    try:
        asyncio.run(run())
    finally:
        engine.shutdown()


if __name__ == "__main__":
    main()
