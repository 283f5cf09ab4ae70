"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory when they need attention (code inside
another runtime's callback, a process whose memory is fully committed, a latency-critical loop), so this
variant keeps the split-KV scratch inside the library.  It must give the same numbers as the regular entry
point, on consecutive calls that reuse the same internal scratch.
"""
import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, ns, hq, hk, d, max_ctx):
    from sonar_b200.layers.attention import AttentionMetadata
    g = torch.Generator().manual_seed(seed)
    ctx = [int(torch.randint(1, max_ctx, (1,), generator=g)) for _ in range(ns)]
    need = sum(-(-c // 16) for c in ctx)
    cache = (torch.randn(need + 3, 2, hk, 16, d, generator=g) * 0.5).to("cuda", torch.bfloat16)
    perm = torch.randperm(need + 2, generator=g)[:need] + 1
    bt = torch.zeros(ns, max(-(-c // 16) for c in ctx), dtype=torch.int32)
    off = 0
    for i, c in enumerate(ctx):
        nb = -(-c // 16)
        bt[i, :nb] = perm[off:off + nb].int()
        off += nb
    q = torch.randn(ns, hq, d, generator=g).to("cuda", torch.bfloat16)
    meta = AttentionMetadata(
        num_tokens=ns, num_seqs=ns, positions=None, slot_mapping=None, block_tables=bt.cuda(),
        seq_lens=torch.tensor(ctx, dtype=torch.int32, device="cuda"),
        query_start_loc=torch.arange(ns + 1, dtype=torch.int32, device="cuda"), max_query_len=1,
        max_seq_len=max(ctx), query_lens_cpu=[1] * ns, seq_lens_cpu=ctx)
    return q, cache, meta


def test_static_scratch_decode_attention_matches_regular_entry_point():
    from sonar_b200.ops import cuda as cu
    fn = cu.lib.sonar_decode_attention_static
    fn.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_long, c_int, c_int,
                   c_int, c_float, c_int, c_int, c_void_p]
    fn.restype = c_int
    stream = torch.cuda.current_stream().cuda_stream
    hq, hk, d = 8, 2, 128
    scale = d ** -0.5
    # two calls in a row with different shapes and split counts: the second reuses the scratch of the first
    for seed, ns, splits, max_ctx in ((1, 5, 4, 3000), (2, 3, 7, 900)):
        q, cache, meta = _case(seed, ns, hq, hk, d, max_ctx)
        want = cu.paged_attention(q, cache, meta, scale)
        got = torch.empty_like(want)
        rc = fn(q.data_ptr(), q.stride(0), cache.data_ptr(), meta.block_tables.data_ptr(), meta.block_tables.stride(0),
                meta.seq_lens.data_ptr(), ns, got.data_ptr(), got.stride(0), hq, hk, d, scale, splits, 0, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs()
        assert (err <= 2e-2 + 2e-2 * want.float().abs()).all(), err.max()
    # over the compiled-in limits: refused, nothing launched
    q, cache, meta = _case(3, 4, hq, hk, d, 100)
    out = torch.empty(4, hq * d, dtype=torch.bfloat16, device="cuda")
    assert fn(q.data_ptr(), q.stride(0), cache.data_ptr(), meta.block_tables.data_ptr(), meta.block_tables.stride(0),
              meta.seq_lens.data_ptr(), 257, out.data_ptr(), out.stride(0), hq, hk, d, scale, 1, 0, stream) == 3
    assert fn(q.data_ptr(), q.stride(0), cache.data_ptr(), meta.block_tables.data_ptr(), meta.block_tables.stride(0),
              meta.seq_lens.data_ptr(), 200, out.data_ptr(), out.stride(0), hq, hk, d, scale, 32, 0, stream) == 3
