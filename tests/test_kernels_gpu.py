"""Numerics of every CUDA kernel against the plain PyTorch fp32 restatement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from sonar_b200.layers.attention import AttentionMetadata  # noqa: E402
from sonar_b200.ops import torch_ref as ref  # noqa: E402


@pytest.fixture(scope="module")
def cu():
    from sonar_b200.ops import cuda
    return cuda


DEV = "cuda"


def _close(a, b, atol, rtol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bad.any(), f"max err {err.max().item():.4g} (tol {atol}+{rtol}·|ref|), {int(bad.sum())} / {bad.numel()} off"


@pytest.mark.parametrize("hidden", [256, 1024, 4096, 8192])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rms_norm(cu, hidden, dtype):
    torch.manual_seed(0)
    x = torch.randn(37, hidden, device=DEV, dtype=dtype)
    w = (torch.rand(hidden, device=DEV) + 0.5).to(dtype)
    want = ref.rms_norm(x.float(), w.float(), 1e-5)
    got = cu.rms_norm(x, w, 1e-5)
    _close(got, want, 2e-2, 1e-2)


@pytest.mark.parametrize("hidden", [1024, 4096])
def test_fused_add_rms_norm(cu, hidden):
    torch.manual_seed(1)
    x = torch.randn(65, hidden, device=DEV, dtype=torch.bfloat16)
    r = torch.randn(65, hidden, device=DEV, dtype=torch.bfloat16)
    w = (torch.rand(hidden, device=DEV) + 0.5).to(torch.bfloat16)
    want_y, want_r = ref.fused_add_rms_norm(x, r, w, 1e-6)
    xy, rr = x.clone(), r.clone()
    cu.fused_add_rms_norm(xy, rr, w, 1e-6)
    _close(rr, want_r, 1e-6, 0)          # residual add is exact in bf16
    _close(xy, want_y, 3e-2, 1e-2)


def test_silu_and_mul(cu):
    torch.manual_seed(2)
    x = torch.randn(50, 2 * 1536, device=DEV, dtype=torch.bfloat16)
    want = ref.silu_and_mul(x.float())
    got = cu.silu_and_mul(x)
    _close(got, want, 2e-2, 1e-2)


@pytest.mark.parametrize("qk_norm", [False, True])
@pytest.mark.parametrize("head_dim", [128, 64])
def test_rope_and_cache(cu, qk_norm, head_dim):
    torch.manual_seed(3)
    t, hq, hk, bs, nblocks = 45, 8, 2, 16, 12
    qkv = torch.randn(t, (hq + 2 * hk) * head_dim, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (t,), device=DEV, dtype=torch.int64)
    cs = ref.build_cos_sin_cache(head_dim, 512, 1e4, None, DEV)
    slots = torch.randperm(nblocks * bs, device=DEV)[:t].int()
    slots[5] = -1
    qw = (torch.rand(head_dim, device=DEV) + 0.5).to(torch.bfloat16) if qk_norm else None
    kw = (torch.rand(head_dim, device=DEV) + 0.5).to(torch.bfloat16) if qk_norm else None
    cache_ref = torch.zeros(nblocks, 2, hk, bs, head_dim, device=DEV, dtype=torch.bfloat16)
    cache = cache_ref.clone()
    q, k, v = qkv.float().split([hq * head_dim, hk * head_dim, hk * head_dim], dim=-1)
    if qk_norm:
        q_ref, k_ref = ref.qk_norm_rope(q, k, qw.float(), kw.float(), 1e-6, pos, cs, head_dim)
    else:
        q_ref, k_ref = ref.rope(q, k, pos, cs, head_dim)
    ref.reshape_and_cache(k_ref.reshape(t, hk, head_dim), v.reshape(t, hk, head_dim), cache_ref, slots)
    work = qkv.clone()
    cu.rope_and_cache(work, pos, cs, cache, slots, hq, hk, head_dim, qw, kw, 1e-6, 1.0, 1.0)
    _close(work[:, : hq * head_dim], q_ref, 4e-2, 2e-2)
    _close(cache, cache_ref, 4e-2, 2e-2)


@pytest.mark.parametrize("head_dim,rot", [(128, 64), (64, 32), (128, 32)])
@pytest.mark.parametrize("qk_norm", [False, True])
def test_rope_partial_rotary(cu, head_dim, rot, qk_norm):
    """Only the pairs below rot/2 turn; the other channels of both halves pass through (and are still normed
    and written to the cache)."""
    torch.manual_seed(4)
    t, hq, hk, bs, nblocks = 37, 4, 2, 16, 8
    qkv = torch.randn(t, (hq + 2 * hk) * head_dim, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 300, (t,), device=DEV, dtype=torch.int64)
    cs = ref.build_cos_sin_cache(rot, 512, 1e4, None, DEV)
    slots = torch.randperm(nblocks * bs, device=DEV)[:t].int()
    qw = (torch.rand(head_dim, device=DEV) + 0.5).to(torch.bfloat16) if qk_norm else None
    kw = (torch.rand(head_dim, device=DEV) + 0.5).to(torch.bfloat16) if qk_norm else None
    cache_ref = torch.zeros(nblocks, 2, hk, bs, head_dim, device=DEV, dtype=torch.bfloat16)
    cache = cache_ref.clone()
    q, k, v = qkv.float().split([hq * head_dim, hk * head_dim, hk * head_dim], dim=-1)
    if qk_norm:
        q_ref, k_ref = ref.qk_norm_rope(q, k, qw.float(), kw.float(), 1e-6, pos, cs, head_dim)
    else:
        q_ref, k_ref = ref.rope(q, k, pos, cs, head_dim)
    ref.reshape_and_cache(k_ref.reshape(t, hk, head_dim), v.reshape(t, hk, head_dim), cache_ref, slots)
    work = qkv.clone()
    cu.rope_and_cache(work, pos, cs, cache, slots, hq, hk, head_dim, qw, kw, 1e-6, 1.0, 1.0)
    _close(work[:, : hq * head_dim], q_ref, 4e-2, 2e-2)
    _close(cache, cache_ref, 4e-2, 2e-2)
    if not qk_norm:      # pass-through channels are bit-identical
        half, rh = head_dim // 2, rot // 2
        got = work[:, : hq * head_dim].reshape(t, hq, head_dim)
        src = qkv[:, : hq * head_dim].reshape(t, hq, head_dim)
        assert torch.equal(got[..., rh:half], src[..., rh:half]) and torch.equal(got[..., half + rh:], src[..., half + rh:])


def _make_attn_case(q_lens, ctx_lens, hq, hk, d, seed=0, nblocks=None):
    torch.manual_seed(seed)
    bs = 16
    ns = len(q_lens)
    need = sum(-(-c // bs) for c in ctx_lens)
    nblocks = nblocks or need + 4
    cache = torch.randn(nblocks, 2, hk, bs, d, device=DEV, dtype=torch.bfloat16) * 0.5
    perm = torch.randperm(nblocks - 1)[:need] + 1
    max_b = max(-(-c // bs) for c in ctx_lens)
    bt = torch.zeros(ns, max_b, dtype=torch.int32)
    off = 0
    for i, c in enumerate(ctx_lens):
        nb = -(-c // bs)
        bt[i, :nb] = perm[off:off + nb].int()
        off += nb
    t = sum(q_lens)
    q = torch.randn(t, hq, d, device=DEV, dtype=torch.bfloat16)
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    meta = AttentionMetadata(
        num_tokens=t, num_seqs=ns, positions=None, slot_mapping=None, block_tables=bt.to(DEV),
        seq_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), query_start_loc=qsl,
        max_query_len=max(q_lens), max_seq_len=max(ctx_lens), query_lens_cpu=q_lens, seq_lens_cpu=ctx_lens)
    return q, cache, meta


ATTN_CASES = [
    ([1, 1, 1], [17, 300, 1025], 8, 2, 128),               # decode, GQA 4
    ([1] * 5, [5, 16, 31, 64, 700], 32, 8, 128),           # decode, llama-8b head layout
    ([1, 1], [40, 90], 8, 1, 128),                         # decode, GQA 8 (70B TP8 shard)
    ([33, 7, 128], [33, 50, 400], 8, 2, 128),              # prefill, chunked (ctx > q)
    ([1, 200, 1, 64], [130, 200, 9, 1000], 8, 2, 128),     # mixed
    ([2, 3], [60, 70], 4, 2, 64),                          # head_dim 64, short multi-token (spec decode shape)
    ([1], [5000], 8, 2, 128),                              # long context, single sequence → split-KV
    ([33, 7, 128], [33, 50, 400], 32, 4, 128),             # prefill, GQA 8 (Qwen3-30B-A3B head layout)
    ([2, 1, 2, 600], [100, 50, 70, 600], 32, 4, 128),      # GQA 8: two-token decode rows (16 per item) + prefill
    ([1] * 40, [513 + 7 * i for i in range(40)], 32, 4, 128),   # GQA 8 decode batch
]


@pytest.mark.parametrize("q_lens,ctx_lens,hq,hk,d", ATTN_CASES)
def test_paged_attention(cu, q_lens, ctx_lens, hq, hk, d):
    q, cache, meta = _make_attn_case(q_lens, ctx_lens, hq, hk, d)
    scale = d ** -0.5
    want = ref.paged_attention(q.float(), cache.float(), meta.block_tables, meta.seq_lens, meta.query_start_loc, scale)
    got = cu.paged_attention(q, cache, meta, scale)
    _close(got.view(-1, hq, d), want, 2e-2, 2e-2)


def test_paged_attention_sliding_window(cu):
    q, cache, meta = _make_attn_case([1, 70], [300, 200], 8, 2, 128, seed=4)
    scale = 128 ** -0.5
    want = ref.paged_attention(q.float(), cache.float(), meta.block_tables, meta.seq_lens, meta.query_start_loc, scale,
                               sliding_window=64)
    got = cu.paged_attention(q, cache, meta, scale, sliding_window=64)
    _close(got.view(-1, 8, 128), want, 2e-2, 2e-2)


def test_paged_attention_strided_q(cu):
    """q as a view into packed qkv rows (the layout the model uses)."""
    q, cache, meta = _make_attn_case([1, 40], [100, 40], 8, 2, 128, seed=5)
    t = q.shape[0]
    packed = torch.randn(t, (8 + 4) * 128, device=DEV, dtype=torch.bfloat16)
    packed[:, : 8 * 128] = q.reshape(t, -1)
    qv = packed.as_strided((t, 8, 128), (packed.stride(0), 128, 1))
    scale = 128 ** -0.5
    want = ref.paged_attention(q.float(), cache.float(), meta.block_tables, meta.seq_lens, meta.query_start_loc, scale)
    got = cu.paged_attention(qv, cache, meta, scale)
    _close(got.view(-1, 8, 128), want, 2e-2, 2e-2)


GEMM_SHAPES = [
    (128, 256, 64), (128, 256, 256), (1, 64, 64), (7, 4096, 4096), (300, 6144, 4096), (1280, 4096, 1024),
    (129, 1024, 8), (256, 128256 // 8, 512), (2048, 2048, 14336 // 8), (33, 72, 136),
]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("bn", [0, 64, 128, 256])
def test_gemm_bf16(cu, m, n, k, bn):
    torch.manual_seed(m * 7 + n + k)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * (1.0 / math.sqrt(k))
    want = x.float() @ w.float().t()
    got = cu.gemm(x, w, force_bn=bn)
    torch.cuda.synchronize()
    cu.check_device_errors()
    _close(got, want, 3e-2, 2e-2)


def test_gemm_fp32_out_bias_fp16(cu):
    torch.manual_seed(9)
    x = torch.randn(100, 512, device=DEV, dtype=torch.float16)
    w = torch.randn(264, 512, device=DEV, dtype=torch.float16) * 0.05
    b = torch.randn(264, device=DEV, dtype=torch.float16)
    _close(cu.gemm(x, w, b), x.float() @ w.float().t() + b.float(), 3e-2, 2e-2)
    _close(cu.gemm(x, w, out_dtype=torch.float32), x.float() @ w.float().t(), 2e-3, 2e-3)
    cu.check_device_errors()


def test_gemm_strided_rows(cu):
    torch.manual_seed(10)
    big = torch.randn(64, 1024, device=DEV, dtype=torch.bfloat16)
    x = big[:, 256:768]                     # row pitch 1024, 512 columns, 16-byte aligned start
    w = torch.randn(128, 512, device=DEV, dtype=torch.bfloat16) * 0.05
    _close(cu.gemm(x, w), x.float() @ w.float().t(), 3e-2, 2e-2)
    cu.check_device_errors()


def test_argmax(cu):
    torch.manual_seed(11)
    logits = torch.randn(33, 128256, device=DEV)
    assert torch.equal(cu.argmax(logits), logits.argmax(-1))


def test_sample_matches_reference_with_shared_noise(cu):
    torch.manual_seed(12)
    b, v = 24, 5000
    logits = torch.randn(b, v, device=DEV) * 3
    noise = torch.empty(b, v, device=DEV).exponential_()
    temp = torch.tensor([0.0, 1.0, 0.7, 1.3] * 6, device=DEV)
    top_k = torch.tensor([0, 0, 50, 0, 7, 1] * 4, device=DEV, dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.9, 0.5, 1.0, 0.8, 0.95] * 3, device=DEV)
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.05, 0.0, 0.2, 0.0] * 2, device=DEV)
    want = ref.sample_from_logits(logits, temp, top_k, top_p, min_p, noise)
    got = cu.sample(logits, temp, top_k, top_p, min_p, noise=noise)
    assert torch.equal(got, want), f"rows differ: {(got != want).nonzero().flatten().tolist()}"


def test_sample_rng_statistics(cu):
    """Without supplied noise the built-in RNG must reproduce the categorical distribution."""
    torch.manual_seed(13)
    v, n = 16, 4096
    row = torch.randn(v, device=DEV) * 1.5
    logits = row[None].repeat(n, 1).contiguous()
    temp = torch.ones(n, device=DEV)
    ids = cu.sample(logits, temp, None, None, None)
    freq = torch.bincount(ids, minlength=v).float() / n
    p = torch.softmax(row, -1)
    assert (freq - p).abs().max() < 0.03
    ids2 = cu.sample(logits, temp, None, None, None)
    assert not torch.equal(ids, ids2)       # successive calls draw fresh noise


@pytest.mark.parametrize("e,k,dtype", [(128, 8, torch.float32), (8, 2, torch.bfloat16), (60, 4, torch.float32)])
def test_topk_softmax_routing(cu, e, k, dtype):
    torch.manual_seed(20)
    logits = (torch.randn(77, e, device=DEV) * 2).to(dtype)
    w_ref, i_ref = ref.topk_softmax(logits.float(), k, True)
    w, i = cu.topk_softmax(logits, k, True)
    assert torch.equal(i.long().sort(-1).values, i_ref.long().sort(-1).values)
    _close(w.gather(1, i.long().argsort(-1)), w_ref.gather(1, i_ref.long().argsort(-1)), 1e-4, 1e-3)


def test_grouped_topk_routing(cu):
    torch.manual_seed(21)
    t, e = 50, 256
    logits = torch.randn(t, e, device=DEV)
    bias = torch.randn(e, device=DEV) * 0.1
    w_ref, i_ref = ref.grouped_topk(logits, bias, 8, 8, 4, True, 2.5, "sigmoid")
    w, i = cu.grouped_topk(logits, bias, 8, 8, 4, True, 2.5, "sigmoid")
    assert torch.equal(i.long().sort(-1).values, i_ref.long().sort(-1).values)
    _close(w.sum(-1), w_ref.sum(-1), 1e-4, 1e-4)


@pytest.mark.parametrize("t,e,k,h,inter,ep", [(200, 8, 2, 256, 128, False), (33, 16, 4, 512, 256, True), (1, 8, 2, 256, 64, False)])
def test_fused_experts(cu, t, e, k, h, inter, ep):
    torch.manual_seed(22)
    x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
    w13 = torch.randn(e, 2 * inter, h, device=DEV, dtype=torch.bfloat16) * 0.05
    w2 = torch.randn(e, h, inter, device=DEV, dtype=torch.bfloat16) * 0.05
    logits = torch.randn(t, e, device=DEV)
    tw, ids = ref.topk_softmax(logits, k, True)
    emap = None
    if ep:   # this "rank" holds the odd experts only
        emap = torch.full((e,), -1, dtype=torch.int32, device=DEV)
        emap[1::2] = torch.arange(e // 2, dtype=torch.int32, device=DEV)
        w13, w2 = w13[1::2].contiguous(), w2[1::2].contiguous()
    want = ref.fused_experts(x.float(), w13.float(), w2.float(), tw, ids, emap)
    got = cu.fused_experts(x, w13, w2, tw, ids, emap)
    torch.cuda.synchronize()
    cu.check_device_errors()
    _close(got, want, 3e-2, 3e-2)


def test_per_token_group_quant_fp8(cu):
    torch.manual_seed(30)
    x = torch.randn(70, 1024, device=DEV, dtype=torch.bfloat16) * 3
    q_ref, s_ref = ref.per_token_group_quant_fp8(x)
    q, s = cu.per_token_group_quant_fp8(x)
    _close(s, s_ref, 1e-7, 1e-5)
    deq = q.float().reshape(70, 8, 128) * s[..., None]
    _close(deq.reshape(70, 1024), x, 0.02, 0.07)     # e4m3: 3 mantissa bits
    assert (q.float() - q_ref.float()).abs().max() <= 32   # at most one fp8 step at the top binade


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (300, 1024, 512), (1, 256, 4096), (1000, 6144, 1024), (77, 136, 256)])
def test_gemm_fp8_block(cu, m, n, k):
    torch.manual_seed(31 + m)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * (k ** -0.5)
    wq, ws = ref.block_quant_fp8_weight(w)
    xq, xs = cu.per_token_group_quant_fp8(x)
    want = ref.gemm_fp8_block(xq, xs.contiguous(), wq, ws, torch.float32)
    got = cu.gemm_fp8_block(xq, xs, wq, ws)
    torch.cuda.synchronize()
    cu.check_device_errors()
    _close(got, want, 2e-2, 2e-2)
    exact = x.float() @ w.float().t()                      # and it approximates the unquantised product
    assert (got.float() - exact).norm() / exact.norm() < 0.06


@pytest.mark.parametrize("q_lens,ctx_lens", [([1, 1, 1], [17, 300, 1025]), ([33, 1, 128], [33, 500, 400]), ([1], [5000])])
def test_paged_attention_fp8_kv_cache(cu, q_lens, ctx_lens):
    q, cache, meta = _make_attn_case(q_lens, ctx_lens, 8, 2, 128, seed=6)
    k_scale, v_scale = 0.02, 0.015
    c8 = torch.empty_like(cache, dtype=torch.float8_e4m3fn)
    c8[:, 0] = (cache[:, 0].float() / k_scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    c8[:, 1] = (cache[:, 1].float() / v_scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    scale = 128 ** -0.5
    want = ref.paged_attention(q.float(), c8, meta.block_tables, meta.seq_lens, meta.query_start_loc, scale,
                               k_scale=k_scale, v_scale=v_scale)
    got = cu.paged_attention(q, c8, meta, scale, k_scale=k_scale, v_scale=v_scale)
    _close(got.view(-1, 8, 128), want, 2e-2, 2e-2)


def test_rope_and_cache_fp8(cu):
    torch.manual_seed(7)
    t, hq, hk, d = 20, 4, 2, 128
    qkv = torch.randn(t, (hq + 2 * hk) * d, device=DEV, dtype=torch.bfloat16)
    pos = torch.arange(t, device=DEV, dtype=torch.int64)
    cs = ref.build_cos_sin_cache(d, 64, 1e4, None, DEV)
    slots = torch.arange(t, device=DEV, dtype=torch.int32) + 16
    cache_ref = torch.zeros(4, 2, hk, 16, d, device=DEV, dtype=torch.float8_e4m3fn)
    cache = cache_ref.clone()
    q, k, v = qkv.float().split([hq * d, hk * d, hk * d], dim=-1)
    _, k_ref = ref.rope(q, k, pos, cs, d)
    ref.reshape_and_cache(k_ref.reshape(t, hk, d), v.reshape(t, hk, d), cache_ref, slots, 0.05, 0.04)
    cu.rope_and_cache(qkv.clone(), pos, cs, cache, slots, hq, hk, d, None, None, 1e-6, 0.05, 0.04)
    assert (cache.float() - cache_ref.float()).abs().max() <= 32    # at most one e4m3 step (bf16 rounding of k before quantising)
    assert ((cache.float() - cache_ref.float()).abs() > 0).float().mean() < 0.05


def _mla_case(q_lens, ctx_lens, h, extra=0, seed=0):
    torch.manual_seed(seed)
    bs, r, pdim = 16, 512, 64
    ns = len(q_lens)
    need = sum(-(-c // bs) for c in ctx_lens)
    cache = (torch.randn(need + 3, bs, r + pdim + extra, device=DEV) * 0.3).to(torch.bfloat16)
    perm = torch.randperm(need + 2)[:need] + 1
    bt = torch.zeros(ns, max(-(-c // bs) for c in ctx_lens), dtype=torch.int32)
    off = 0
    for i, c in enumerate(ctx_lens):
        nb = -(-c // bs)
        bt[i, :nb] = perm[off:off + nb].int()
        off += nb
    t = sum(q_lens)
    q_lat = (torch.randn(t, h, r, device=DEV) * 0.3).to(torch.bfloat16)
    q_pe = (torch.randn(t, h, pdim, device=DEV) * 0.3).to(torch.bfloat16)
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(c - q, c) for q, c in zip(q_lens, ctx_lens)]).to(DEV)
    meta = AttentionMetadata(num_tokens=t, num_seqs=ns, positions=pos, slot_mapping=None, block_tables=bt.to(DEV),
                             seq_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), query_start_loc=qsl,
                             max_query_len=max(q_lens), max_seq_len=max(ctx_lens), query_lens_cpu=q_lens,
                             seq_lens_cpu=ctx_lens)
    return q_lat, q_pe, cache, meta


@pytest.mark.parametrize("q_lens,ctx_lens,h,extra", [([1, 1], [37, 600], 16, 0), ([5, 1, 40], [5, 130, 300], 24, 128),
                                                     ([1], [4000], 16, 0)])
def test_mla_attention_dense(cu, q_lens, ctx_lens, h, extra):
    q_lat, q_pe, cache, meta = _mla_case(q_lens, ctx_lens, h, extra)
    scale = 576 ** -0.5
    want = ref.mla_paged_attention(q_lat.float(), q_pe.float(), cache.float(), meta.block_tables, meta.seq_lens,
                                   meta.query_start_loc, scale, 512, None, 64)
    got = cu.mla_paged_attention(q_lat, q_pe, cache, meta, scale, 512, None, 64)
    _close(got, want, 2e-2, 2e-2)


def test_mla_attention_sparse_topk(cu):
    q_lat, q_pe, cache, meta = _mla_case([1, 3], [500, 900], 16, 128, seed=3)
    t = q_lat.shape[0]
    k = 64
    topk = torch.full((t, k), -1, dtype=torch.int32, device=DEV)
    pos = meta.positions.tolist()
    g = torch.Generator().manual_seed(0)
    for i in range(t):
        n = min(k - 5, pos[i] + 1)
        topk[i, :n] = torch.randperm(pos[i] + 1, generator=g)[:n].int().to(DEV)
    scale = 576 ** -0.5
    want = ref.mla_paged_attention(q_lat.float(), q_pe.float(), cache.float(), meta.block_tables, meta.seq_lens,
                                   meta.query_start_loc, scale, 512, topk, 64)
    got = cu.mla_paged_attention(q_lat, q_pe, cache, meta, scale, 512, topk, 64)
    _close(got, want, 2e-2, 2e-2)


def test_mla_cache_write(cu):
    torch.manual_seed(4)
    t = 30
    kv_c = torch.randn(t, 512, device=DEV, dtype=torch.bfloat16)
    rest = torch.randn(t, 64 + 128, device=DEV, dtype=torch.bfloat16)
    slots = torch.randperm(64, device=DEV)[:t].int()
    slots[3] = -1
    want = torch.zeros(4, 16, 704, device=DEV, dtype=torch.bfloat16)
    got = want.clone()
    ref.mla_cache_write(kv_c, rest, want, slots)
    cu.mla_cache_write(kv_c, rest, got, slots)
    assert torch.equal(got, want)


@pytest.mark.parametrize("bucket,n_seqs", [(1, 1), (2, 2), (4, 3), (8, 8), (16, 11), (32, 32), (64, 50), (80, 80)])
@pytest.mark.parametrize("hq,hk", [(32, 4), (32, 8)])
def test_decode_attention_graph_bucket_geometry(cu, bucket, n_seqs, hq, hk):
    """Decode steps replayed from a CUDA graph use a grid and a KV split count fixed by the padded batch size;
    surplus slots exit on the device-side count.  Same numbers as the PyTorch restatement."""
    ctx = [513 + (37 * i) % 255 for i in range(n_seqs)]
    q, cache, meta = _make_attn_case([1] * n_seqs, ctx, hq, hk, 128, seed=bucket)
    cu.build_attention_work(meta, None, hq // hk, hk, graph_bucket=bucket)
    got = cu.paged_attention(q, cache, meta, 128 ** -0.5)
    torch.cuda.synchronize()
    want = ref.paged_attention(q.float(), cache.float(), meta.block_tables, meta.seq_lens, meta.query_start_loc,
                               128 ** -0.5)
    _close(got.view(-1, hq, 128), want, 2e-2, 2e-2)


def test_bounded_wait_reports_instead_of_hanging(cu):
    """Failure detection on the device: a kernel waiting for a peer flag that nothing ever sets gives up after
    its time limit, records the wait site in the device error word and returns — the context stays usable
    and the host sees the error.  (A flag word that stays 0 stands in for a peer that died between steps.)"""
    import time
    flags = torch.zeros(4, dtype=torch.int32, device=DEV)         # 2 row blocks × tp 2, never published
    err = cu.error_word(torch.device(DEV))
    torch.cuda.synchronize()
    t0 = time.time()
    cu.tp_wait(flags, 2, 128, 256, 7, None, err)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.0 < waited < 10.0, waited                             # the 2 s limit, not forever
    with pytest.raises(RuntimeError, match="peer flag"):
        cu.check_device_errors()
    cu.check_device_errors()                                       # the word was cleared: no stale error
    # the context is still usable and a published flag lets the same kernel through immediately
    flags.fill_(7)
    cu.tp_wait(flags, 2, 128, 256, 7, None, err)
    torch.cuda.synchronize()
    cu.check_device_errors()
    assert float(torch.ones(4, device=DEV).sum()) == 4.0
