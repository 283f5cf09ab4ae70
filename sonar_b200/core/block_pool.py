"""Paged KV-cache block pool with prefix caching.

Design: blocks are integers.  All per-block state lives in flat Python lists
indexed by block id (reference count, hash, intrusive doubly-linked free list),
so allocation, release and mid-list removal are O(1) with no per-block object.
Freed blocks keep their hash and stay findable until they are handed out
again; the free list is ordered least-recently-freed first, and a request's
blocks are released tail-first so the deepest prefix blocks are evicted first.

Parity: ``aphrodite/v1/core/block_pool.py:141-700`` (``get_cached_block``,
``cache_full_blocks``, ``get_new_blocks``, ``touch``, ``free_blocks``,
``reset_prefix_cache``) and the free queue of ``v1/core/kv_cache_utils.py:182``.
"""
from __future__ import annotations

import hashlib
import struct
from typing import Callable, Iterable, Sequence

NULL_BLOCK = 0  # block 0 is a permanent placeholder (never allocated, never freed)
_NIL = -1


class KVEvent:
    __slots__ = ("kind", "block_hashes", "parent_hash", "token_ids")

    def __init__(self, kind: str, block_hashes: list[bytes], parent_hash: bytes | None = None,
                 token_ids: list[int] | None = None) -> None:
        self.kind, self.block_hashes, self.parent_hash, self.token_ids = kind, block_hashes, parent_hash, token_ids

    def __repr__(self) -> str:
        return f"KVEvent({self.kind}, n={len(self.block_hashes)})"


class BlockPool:
    def __init__(self, num_blocks: int, enable_caching: bool = True, collect_events: bool = False) -> None:
        if num_blocks < 2:
            raise ValueError("the pool needs at least 2 blocks (one is the null block)")
        self.num_blocks = num_blocks
        self.enable_caching = enable_caching
        self.ref_cnt = [0] * num_blocks
        self.block_hash: list[bytes | None] = [None] * num_blocks
        # intrusive free list: head/tail sentinels are virtual
        self._prev = [_NIL] * num_blocks
        self._next = [_NIL] * num_blocks
        self._in_free = [False] * num_blocks
        self._head = _NIL
        self._tail = _NIL
        self.num_free = 0
        for b in range(1, num_blocks):
            self._push_back(b)
        self.ref_cnt[NULL_BLOCK] = 1
        self.hash_to_block: dict[bytes, int] = {}
        self.collect_events = collect_events
        self.events: list[KVEvent] = []
        self.on_evict = None          # callable(block id, hash): a lower tier that keeps evicted blocks

    # ---- free list -----------------------------------------------------
    def _push_back(self, b: int) -> None:
        self._prev[b] = self._tail
        self._next[b] = _NIL
        if self._tail != _NIL:
            self._next[self._tail] = b
        else:
            self._head = b
        self._tail = b
        self._in_free[b] = True
        self.num_free += 1

    def _unlink(self, b: int) -> None:
        p, n = self._prev[b], self._next[b]
        if p != _NIL:
            self._next[p] = n
        else:
            self._head = n
        if n != _NIL:
            self._prev[n] = p
        else:
            self._tail = p
        self._prev[b] = self._next[b] = _NIL
        self._in_free[b] = False
        self.num_free -= 1

    def free_list(self) -> list[int]:
        out, b = [], self._head
        while b != _NIL:
            out.append(b)
            b = self._next[b]
        return out

    # ---- public API ----------------------------------------------------
    def get_num_free_blocks(self) -> int:
        return self.num_free

    def get_usage(self) -> float:
        total = self.num_blocks - 1
        return 1.0 - self.num_free / total if total else 0.0

    def get_cached_block(self, block_hash: bytes) -> int | None:
        return self.hash_to_block.get(block_hash)

    def get_new_blocks(self, n: int) -> list[int]:
        if n > self.num_free:
            raise ValueError(f"cannot allocate {n} blocks, only {self.num_free} free")
        out = []
        for _ in range(n):
            b = self._head
            self._unlink(b)
            self._maybe_evict(b)
            self.ref_cnt[b] = 1
            out.append(b)
        return out

    def _maybe_evict(self, b: int) -> None:
        h = self.block_hash[b]
        if h is None:
            return
        if self.hash_to_block.get(h) == b:
            del self.hash_to_block[h]
            if self.on_evict is not None:
                self.on_evict(b, h)
            if self.collect_events:
                self.events.append(KVEvent("removed", [h]))
        self.block_hash[b] = None

    def touch(self, blocks: Iterable[int]) -> None:
        """Take a reference on cached blocks (a prefix hit); blocks that were
        sitting in the free list leave it."""
        for b in blocks:
            if self.ref_cnt[b] == 0 and self._in_free[b]:
                self._unlink(b)
            self.ref_cnt[b] += 1

    def free_blocks(self, blocks: Iterable[int]) -> None:
        """Drop one reference per block, in the order given; blocks reaching
        zero join the tail of the free list in that order."""
        for b in blocks:
            if b == NULL_BLOCK:
                continue
            self.ref_cnt[b] -= 1
            assert self.ref_cnt[b] >= 0, f"double free of block {b}"
            if self.ref_cnt[b] == 0:
                self._push_back(b)

    def cache_full_blocks(self, blocks: Sequence[int], block_hashes: Sequence[bytes],
                          num_cached: int, num_full: int, token_ids: Sequence[int] | None = None,
                          block_size: int = 0) -> None:
        """Publish blocks ``[num_cached, num_full)`` of a request under their
        chained hashes."""
        if not self.enable_caching or num_full <= num_cached:
            return
        new_hashes = []
        for i in range(num_cached, num_full):
            b, h = blocks[i], block_hashes[i]
            if self.block_hash[b] is not None:
                continue
            self.block_hash[b] = h
            # first writer wins; a duplicate block stays private to its owner
            self.hash_to_block.setdefault(h, b)
            new_hashes.append(h)
        if self.collect_events and new_hashes:
            parent = block_hashes[num_cached - 1] if num_cached > 0 else None
            toks = None
            if token_ids is not None and block_size:
                toks = list(token_ids[num_cached * block_size:num_full * block_size])
            self.events.append(KVEvent("stored", new_hashes, parent, toks))

    def reset_prefix_cache(self) -> bool:
        used = self.num_blocks - 1 - self.num_free
        if used:
            return False
        self.hash_to_block.clear()
        self.block_hash = [None] * self.num_blocks
        if self.collect_events:
            self.events.append(KVEvent("cleared", []))
        return True

    def take_events(self) -> list[KVEvent]:
        ev, self.events = self.events, []
        return ev


# ---------------------------------------------------------------------------
# chained block hashing
# ---------------------------------------------------------------------------
_ROOT = b"\x00" * 16


def _sha256_block(parent: bytes, tokens: Sequence[int], extra: bytes) -> bytes:
    h = hashlib.sha256()
    h.update(parent)
    h.update(struct.pack(f"<{len(tokens)}q", *tokens))
    if extra:
        h.update(extra)
    return h.digest()[:16]


def _builtin_block(parent: bytes, tokens: Sequence[int], extra: bytes) -> bytes:
    return struct.pack("<q", hash((parent, tuple(tokens), extra))) * 2


HASH_FNS: dict[str, Callable[[bytes, Sequence[int], bytes], bytes]] = {
    "sha256": _sha256_block, "builtin": _builtin_block}


def make_block_hasher(block_size: int, algo: str = "sha256"):
    """Return ``f(request) -> list[new block hashes]``: hashes of the full
    blocks of ``request.all_token_ids`` not yet in ``request.block_hashes``.
    The key of a block covers its parent's key, its token ids and the extra
    keys (cache salt, LoRA name) — parity ``kv_cache_utils.py:568,655``."""
    fn = HASH_FNS[algo]

    def hasher(req) -> list[bytes]:
        start = len(req.block_hashes) * block_size
        toks = req.all_token_ids
        n = len(toks)
        if start + block_size > n:
            return []
        extra = b""
        if req.cache_salt:
            extra += b"s:" + req.cache_salt.encode()
        if req.lora_name:
            extra += b"l:" + req.lora_name.encode()
        parent = req.block_hashes[-1] if req.block_hashes else _ROOT
        out = []
        while start + block_size <= n:
            parent = fn(parent, toks[start:start + block_size], extra)
            out.append(parent)
            start += block_size
        return out

    return hasher
