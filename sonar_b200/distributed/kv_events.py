"""KV-cache event stream: block stored / removed / cleared events, batched and published on a ZMQ
PUB socket so an external router can mirror which prefixes each engine holds.

Wire format (msgpack): ``[seq: int, payload]`` frames under ``topic``, where payload is
``{"ts": float, "events": [{"type": "stored", "block_hashes": [...], "parent": hash | None,
"token_ids": [...]} | {"type": "removed", "block_hashes": [...]} | {"type": "cleared"}]}``.
A small replay buffer answers ``[start_seq]`` requests on a ROUTER socket so a subscriber that
missed frames can catch up.

Parity: ``aphrodite/distributed/kv_events.py`` (``ZmqEventPublisher``, ``KVEventBatch``, replay).
"""
from __future__ import annotations

import threading
import time
from collections import deque

import msgpack
import zmq

from sonar_b200.logger import init_logger

logger = init_logger(__name__)


def encode_events(events) -> list[dict]:
    out = []
    for e in events:
        d: dict = {"type": e.kind}
        if e.kind != "cleared":
            d["block_hashes"] = [h.hex() if isinstance(h, (bytes, bytearray)) else h for h in e.block_hashes]
        if e.kind == "stored":
            p = getattr(e, "parent", None)
            d["parent"] = p.hex() if isinstance(p, (bytes, bytearray)) else p
            d["token_ids"] = list(getattr(e, "token_ids", None) or [])
        out.append(d)
    return out


class KVEventPublisher:
    def __init__(self, endpoint: str = "tcp://127.0.0.1:0", replay_endpoint: str | None = None,
                 topic: str = "kv-events", buffer_steps: int = 10000) -> None:
        self.ctx = zmq.Context.instance()
        self.pub = self.ctx.socket(zmq.PUB)
        if endpoint.endswith(":0"):
            port = self.pub.bind_to_random_port(endpoint[:-2])
            self.endpoint = f"{endpoint[:-2]}:{port}"
        else:
            self.pub.bind(endpoint)
            self.endpoint = endpoint
        self.topic = topic.encode()
        self.seq = 0
        self.buffer: deque[tuple[int, bytes]] = deque(maxlen=buffer_steps)
        self._lock = threading.Lock()
        self.replay = None
        self._stop = False
        if replay_endpoint:
            self.replay = self.ctx.socket(zmq.ROUTER)
            if replay_endpoint.endswith(":0"):
                port = self.replay.bind_to_random_port(replay_endpoint[:-2])
                self.replay_endpoint = f"{replay_endpoint[:-2]}:{port}"
            else:
                self.replay.bind(replay_endpoint)
                self.replay_endpoint = replay_endpoint
            self._thread = threading.Thread(target=self._serve_replay, daemon=True)
            self._thread.start()

    def publish(self, events) -> int | None:
        """Publish one batch (the events of one scheduler step).  Returns its sequence number."""
        if not events:
            return None
        payload = msgpack.packb({"ts": time.time(), "events": encode_events(events)}, use_bin_type=True)
        with self._lock:
            seq = self.seq
            self.seq += 1
            self.buffer.append((seq, payload))
        self.pub.send_multipart([self.topic, seq.to_bytes(8, "big"), payload])
        return seq

    def _serve_replay(self) -> None:
        poller = zmq.Poller()
        poller.register(self.replay, zmq.POLLIN)
        while not self._stop:
            if not poller.poll(200):
                continue
            frames = self.replay.recv_multipart()
            ident, start = frames[0], int.from_bytes(frames[-1], "big")
            with self._lock:
                items = [(s, p) for s, p in self.buffer if s >= start]
            for s, p in items:
                self.replay.send_multipart([ident, b"", s.to_bytes(8, "big"), p])
            self.replay.send_multipart([ident, b"", (-1 & 0xFFFFFFFFFFFFFFFF).to_bytes(8, "big"), b""])   # end marker

    def close(self) -> None:
        self._stop = True
        self.pub.close(linger=0)
        if self.replay is not None:
            self._thread.join(timeout=1)
            self.replay.close(linger=0)
