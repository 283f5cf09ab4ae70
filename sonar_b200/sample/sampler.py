"""Token sampler.

Fast path (what throughput runs hit): one fused kernel call — arg-max for
greedy rows, temperature + top-k/top-p/min-p + exponential-race sampling for
the rest (``ops.sample``).  Rows that ask for more go through the extended
chain, applied in a fixed order on fp32 logits: DRY → penalties →
no-repeat-ngram → logit bias / allowed ids / bad words / min-tokens →
temperature (dynamic temperature; skipped here when ``temperature_last``) →
top-nσ → top-a → tail-free → η/ε cutoffs → typical-p → quadratic smoothing →
XTC → (mirostat v2, exclusive of the truncation samplers) → skew → late
temperature → top-k/top-p/min-p + draw.

Parity: ``aphrodite/v1/sample/sampler.py:25-40,95,179-193,433`` (chain and
order), ``v1/sample/ops/topk_topp_sampler.py:72`` and
``csrc/libtorch_stable/sampler.cu:14`` (penalties).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from sonar_b200 import ops
from sonar_b200.ops import torch_ref
from sonar_b200.sampling_params import SamplingParams

_EPS = 1e-5


@dataclass
class SamplingMetadata:
    """Per-row controls for one sampling call (row i ↔ ``params[i]``)."""
    params: list[SamplingParams]
    temperature: torch.Tensor
    top_k: torch.Tensor
    top_p: torch.Tensor
    min_p: torch.Tensor
    all_greedy: bool
    all_simple: bool                       # no row needs the extended chain / penalties / masks
    prompt_token_ids: list[list[int]] = field(default_factory=list)
    output_token_ids: list[list[int]] = field(default_factory=list)
    generators: dict[int, torch.Generator] = field(default_factory=dict)
    max_num_logprobs: int | None = None
    mirostat_mu: dict[int, float] = field(default_factory=dict)   # row → mu (updated in place)
    req_ids: list[str] = field(default_factory=list)


@dataclass
class SamplerOutput:
    token_ids: torch.Tensor                                    # [B] int64 on the logits device
    logprobs: list[dict[int, float]] | None = None             # per row: {token: logprob}


def _needs_chain(p: SamplingParams) -> bool:
    return (p.needs_penalties or p.needs_extended or bool(p.logit_bias) or bool(p.allowed_token_ids)
            or bool(p._bad_words_token_ids) or p.min_tokens > 0)


def make_sampling_metadata(params: list[SamplingParams], prompt_ids: list[list[int]],
                           output_ids: list[list[int]], device, generators=None, mirostat_mu=None,
                           req_ids=None) -> SamplingMetadata:
    temps = [0.0 if p.temperature < _EPS else p.temperature for p in params]
    lp = [p.logprobs for p in params if p.logprobs is not None]
    n = len(params)
    # one pinned staging block and one asynchronous copy: a pageable host→device copy would block the host
    # until everything queued on the stream has run, which defeats scheduling ahead of the GPU
    cuda = torch.device(device).type == "cuda"
    stage = torch.empty((4, n), dtype=torch.float32, pin_memory=cuda)
    sv = stage.numpy()
    sv[0] = temps
    sv[1] = [p.top_k for p in params]
    sv[2] = [p.top_p for p in params]
    sv[3] = [p.min_p for p in params]
    dev = stage.to(device, non_blocking=cuda)
    return SamplingMetadata(
        params=params,
        temperature=dev[0],
        top_k=dev[1].to(torch.int32),
        top_p=dev[2],
        min_p=dev[3],
        all_greedy=all(t == 0.0 for t in temps),
        all_simple=not any(_needs_chain(p) for p in params),
        prompt_token_ids=prompt_ids, output_token_ids=output_ids, generators=generators or {},
        max_num_logprobs=(max(lp) if lp else None), mirostat_mu=mirostat_mu if mirostat_mu is not None else {},
        req_ids=req_ids or [])


class Sampler:
    def __call__(self, logits: torch.Tensor, md: SamplingMetadata) -> SamplerOutput:
        raw_logprobs = None
        if md.max_num_logprobs is not None:
            raw_logprobs = torch.log_softmax(logits.float(), dim=-1)
        if md.all_simple:
            if md.all_greedy:
                ids = ops.argmax(logits)
            else:
                ids = ops.sample(logits, md.temperature, md.top_k, md.top_p, md.min_p, generators=md.generators)
        else:
            ids = self._chain(logits.float().clone(), md)
        out = SamplerOutput(token_ids=ids)
        if raw_logprobs is not None:
            out.logprobs = self._gather_logprobs(raw_logprobs, ids, md)
        return out

    # ------------------------------------------------------------------
    def _gather_logprobs(self, lp: torch.Tensor, ids: torch.Tensor, md: SamplingMetadata):
        k = md.max_num_logprobs
        v = lp.shape[-1]
        kk = v if k == -1 else min(max(k, 1), v)
        top_v, top_i = lp.topk(kk, dim=-1)
        chosen = lp.gather(1, ids.long()[:, None])[:, 0]
        top_v, top_i, chosen, ids_l = top_v.tolist(), top_i.tolist(), chosen.tolist(), ids.tolist()
        res: list[dict[int, float]] = []
        for r, p in enumerate(md.params):
            if p.logprobs is None:
                res.append({})
                continue
            n = v if p.logprobs == -1 else p.logprobs
            d = {ids_l[r]: chosen[r]}
            for j in range(min(n, kk)):
                d.setdefault(top_i[r][j], top_v[r][j])
            res.append(d)
        return res

    def _chain(self, logits: torch.Tensor, md: SamplingMetadata) -> torch.Tensor:
        b, v = logits.shape
        dev = logits.device
        P = md.params
        temperature = md.temperature.clone()

        # ---- history-based penalties ----------------------------------
        for r, p in enumerate(P):
            if p.dry_multiplier > 0:
                _apply_dry(logits[r], md.prompt_token_ids[r] + md.output_token_ids[r], p)
        if any(p.needs_penalties for p in P):
            prompt_mask = torch.zeros(b, v, dtype=torch.bool, device=dev)
            counts = torch.zeros(b, v, dtype=torch.int32, device=dev)
            for r, p in enumerate(P):
                if not p.needs_penalties:
                    continue
                if md.prompt_token_ids[r]:
                    prompt_mask[r, torch.tensor(md.prompt_token_ids[r], device=dev).clamp_max(v - 1)] = True
                if md.output_token_ids[r]:
                    t = torch.tensor(md.output_token_ids[r], device=dev).clamp_max(v - 1)
                    counts[r].scatter_add_(0, t, torch.ones_like(t, dtype=torch.int32))
            pres = torch.tensor([p.presence_penalty for p in P], device=dev)
            freq = torch.tensor([p.frequency_penalty for p in P], device=dev)
            rep = torch.tensor([p.repetition_penalty for p in P], device=dev)
            logits = torch_ref.apply_penalties(logits, prompt_mask, counts, pres, freq, rep)
        for r, p in enumerate(P):
            hist = md.prompt_token_ids[r] + md.output_token_ids[r]
            if p.no_repeat_ngram_size > 0:
                n = p.no_repeat_ngram_size
                if len(hist) >= n:
                    tail = tuple(hist[len(hist) - n + 1:]) if n > 1 else ()
                    banned = [hist[i + n - 1] for i in range(len(hist) - n + 1)
                              if tuple(hist[i:i + n - 1]) == tail]
                    if banned:
                        logits[r, torch.tensor(banned, device=dev)] = float("-inf")
            # ---- hard masks ------------------------------------------------
            if p.logit_bias:
                idx = torch.tensor(list(p.logit_bias.keys()), device=dev)
                logits[r, idx] += torch.tensor(list(p.logit_bias.values()), device=dev, dtype=logits.dtype)
            if p.allowed_token_ids:
                keep = torch.zeros(v, dtype=torch.bool, device=dev)
                keep[torch.tensor(p.allowed_token_ids, device=dev)] = True
                logits[r].masked_fill_(~keep, float("-inf"))
            if p._bad_words_token_ids:
                out = md.output_token_ids[r]
                for bw in p._bad_words_token_ids:
                    if len(bw) == 1 or (len(out) >= len(bw) - 1 and out[len(out) - len(bw) + 1:] == bw[:-1]):
                        logits[r, bw[-1]] = float("-inf")
            if p.min_tokens > len(md.output_token_ids[r]):
                stops = set(p.all_stop_token_ids)
                if p._eos_token_id is not None:
                    stops.add(p._eos_token_id)
                if stops:
                    logits[r, torch.tensor(sorted(stops), device=dev)] = float("-inf")

        # ---- temperature ----------------------------------------------
        late_temp = torch.ones(b, device=dev)
        for r, p in enumerate(P):
            if p.dynatemp_max > 0 and temperature[r] > 0:
                pr = torch.softmax(logits[r], dim=-1)
                ent = -(pr * torch.log(pr.clamp_min(1e-10))).sum()
                n_valid = int(torch.isfinite(logits[r]).sum())
                max_ent = math.log(max(n_valid, 2))
                frac = float((ent / max_ent).clamp(0, 1)) ** p.dynatemp_exponent
                temperature[r] = max(p.dynatemp_min + (p.dynatemp_max - p.dynatemp_min) * frac, 1e-2)
            if p.temperature_last and temperature[r] > 0:
                late_temp[r] = temperature[r]
                temperature[r] = 1.0
        greedy = temperature < _EPS
        safe_t = torch.where(greedy, torch.ones_like(temperature), temperature)
        logits = logits / safe_t[:, None]

        # ---- truncation samplers (row-wise; only rows that ask) -----------
        for r, p in enumerate(P):
            if greedy[r]:
                continue
            row = logits[r]
            if p.mirostat_mode == 2:
                mu = md.mirostat_mu.setdefault(r, 2.0 * p.mirostat_tau)
                pr = torch.softmax(row, dim=-1)
                surprise = -torch.log2(pr.clamp_min(1e-30))
                mask = surprise > mu
                mask[row.argmax()] = False
                row.masked_fill_(mask, float("-inf"))
                continue
            if p.nsigma > 0:
                finite = row[torch.isfinite(row)]
                row.masked_fill_(row < row.max() - p.nsigma * finite.std(), float("-inf"))
            if p.top_a > 0:
                pr = torch.softmax(row, dim=-1)
                row.masked_fill_(pr < p.top_a * pr.max() ** 2, float("-inf"))
            if p.tfs < 1.0:
                srt, idx = torch.softmax(row, dim=-1).sort(descending=True)
                d2 = srt.diff().diff().abs()
                d2 = d2 / d2.sum().clamp_min(1e-10)
                cdf = d2.cumsum(0)
                drop = torch.cat([torch.zeros(1, dtype=torch.bool, device=dev), cdf > p.tfs,
                                  torch.ones(1, dtype=torch.bool, device=dev)])
                row[idx[drop]] = float("-inf")
            if p.eta_cutoff > 0 or p.epsilon_cutoff > 0:
                pr = torch.softmax(row, dim=-1)
                thr = 0.0
                if p.epsilon_cutoff > 0:
                    thr = p.epsilon_cutoff * 1e-4
                if p.eta_cutoff > 0:
                    eta = p.eta_cutoff * 1e-4
                    ent = -(pr * torch.log(pr.clamp_min(1e-10))).sum()
                    thr = max(thr, float(min(eta, math.sqrt(eta) * math.exp(-float(ent)))))
                mask = pr < thr
                mask[row.argmax()] = False
                row.masked_fill_(mask, float("-inf"))
            if p.typical_p < 1.0:
                lp = torch.log_softmax(row, dim=-1)
                pr = lp.exp()
                ent = -(pr * torch.where(torch.isfinite(lp), lp, torch.zeros_like(lp))).sum()
                dev_from = (-lp - ent).abs()
                order = dev_from.argsort()
                cum = pr[order].cumsum(0)
                last = int((cum < p.typical_p).sum())
                row[order[last + 1:]] = float("-inf")
            if p.smoothing_factor > 0:
                mx = row.max()
                diff = row - mx
                k = p.smoothing_factor * (3 - p.smoothing_curve) / 2
                s = p.smoothing_factor * (p.smoothing_curve - 1) / 2
                new = -(k * diff ** 2) + (s * diff ** 3) + mx
                logits[r] = torch.where(torch.isfinite(row), new, row)
                row = logits[r]
            if p.xtc_probability > 0:
                gen = md.generators.get(r)
                u = torch.rand((), generator=gen, device=gen.device if gen else "cpu")
                if float(u) < p.xtc_probability:
                    pr = torch.softmax(row, dim=-1)
                    above = (pr >= p.xtc_threshold).nonzero()[:, 0]
                    if above.numel() > 1:
                        keep = above[pr[above].argmin()]
                        drop = above[above != keep]
                        row[drop] = float("-inf")
            if p.skew != 0:
                pr = torch.softmax(row, dim=-1) ** math.exp(p.skew)
                logits[r] = torch.log(pr.clamp_min(1e-38)).masked_fill(~torch.isfinite(row), float("-inf"))
        logits = logits / late_temp[:, None]

        # ---- top-k / top-p / min-p + draw ---------------------------------
        unit_t = torch.where(greedy, torch.zeros_like(temperature), torch.ones_like(temperature))
        ids = torch_ref.sample_from_logits(logits, unit_t, md.top_k, md.top_p, md.min_p, None, md.generators)
        for r, p in enumerate(P):
            if p.mirostat_mode == 2 and not greedy[r]:
                pr = torch.softmax(logits[r], dim=-1)
                surprise = -math.log2(max(float(pr[ids[r]]), 1e-30))
                md.mirostat_mu[r] = md.mirostat_mu[r] - p.mirostat_eta * (surprise - p.mirostat_tau)
        return ids


def _apply_dry(row: torch.Tensor, hist: list[int], p: SamplingParams) -> None:
    """DRY: penalise tokens that would extend a verbatim repeat of the context.
    For every earlier occurrence of the last token, measure how many tokens
    before it match the current tail; the token that followed that occurrence
    gets ``multiplier · base^(match_len − allowed_length)`` subtracted."""
    if p.dry_range > 0:
        hist = hist[-p.dry_range:]
    n = len(hist)
    if n < 2:
        return
    breakers = set(p.dry_sequence_breaker_ids)
    last = hist[-1]
    if last in breakers:
        return
    best: dict[int, int] = {}
    for i in range(n - 2, -1, -1):
        if hist[i] != last:
            continue
        length = 1
        while i - length >= 0 and length < 50:
            a, b = hist[i - length], hist[n - 1 - length]
            if a != b or a in breakers:
                break
            length += 1
        nxt = hist[i + 1]
        if length > best.get(nxt, 0):
            best[nxt] = length
    for tok, length in best.items():
        if length >= p.dry_allowed_length and tok < row.shape[0]:
            row[tok] -= p.dry_multiplier * p.dry_base ** (length - p.dry_allowed_length)
