"""Logits processors used by the tests (importable by qualified name)."""
import torch

from sonar_b200.sample.logits_processor import LogitsProcessor


class ForceToken(LogitsProcessor):
    """Requests that pass ``extra_args={"force_token": t}`` can only emit token t."""
    calls = 0

    def is_active(self, params):
        return bool(params.extra_args and "force_token" in params.extra_args)

    def apply(self, logits, rows):
        type(self).calls += 1
        for i, r in enumerate(rows):
            keep = logits[i, r.params.extra_args["force_token"]].clone()
            logits[i].fill_(float("-inf"))
            logits[i, r.params.extra_args["force_token"]] = keep


class NoImmediateRepeat(LogitsProcessor):
    """Bans the previous output token (needs the token history)."""
    needs_history = True

    def apply(self, logits, rows):
        out = logits.clone()
        for i, r in enumerate(rows):
            if r.output_token_ids:
                out[i, r.output_token_ids[-1]] = float("-inf")
        return out
