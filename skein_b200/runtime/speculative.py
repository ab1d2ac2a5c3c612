"""Speculative decoding loop (Leviathan et al.): a draft model proposes k tokens, the target model scores
all k + 1 positions in one forward, `core.speculative_verify` (C++) keeps the longest accepted prefix and
draws the correction or bonus token. The output distribution equals sampling from the target alone.

`draft_step(seq) -> probs[V]` and `target_probs(seq, k) -> [k + 1][V]` are callables so that the loop works
with the engine's models as well as with the toy distributions of the tests, as in the reference
(crates/skein_runtime/src/speculative.rs:184 `generate` over closures; its runtime path uses
forward_full without KV reuse: distributed/gpu_rank.rs:703,2197).
"""
from __future__ import annotations

import random

from .. import core


def softmax(logits):
    m = max(logits)
    e = [pow(2.718281828459045, x - m) for x in logits]
    s = sum(e)
    return [x / s for x in e]


def generate(prompt, max_new_tokens: int, k: int, draft_step, target_probs, seed: int = 0, sample_draft=None):
    """Returns (generated tokens, stats). stats: proposed, accepted, target_calls."""
    rng = random.Random(seed)
    seq = list(prompt)
    out = []
    stats = {"proposed": 0, "accepted": 0, "target_calls": 0}
    while len(out) < max_new_tokens:
        kk = min(k, max_new_tokens - len(out) - 1) if max_new_tokens - len(out) > 1 else 0
        draft_tokens, draft_ps = [], []
        cur = list(seq)
        for _ in range(kk):
            q = draft_step(cur)
            t = sample_draft(q, rng) if sample_draft else core_sample(q, rng.random())
            draft_tokens.append(t)
            draft_ps.append(list(q))
            cur.append(t)
        ps = target_probs(seq, draft_tokens)
        stats["target_calls"] += 1
        uniforms = [rng.random() for _ in range(kk + 1)]
        accepted, correction = core.speculative_verify(draft_tokens, draft_ps, [list(p) for p in ps], uniforms)
        stats["proposed"] += kk
        stats["accepted"] += len(accepted)
        new = list(accepted) + [correction]
        new = new[: max_new_tokens - len(out)]
        out.extend(new)
        seq.extend(new)
    return out, stats


def core_sample(dist, u: float) -> int:
    run = 0.0
    for i, p in enumerate(dist):
        run += p
        if u < run:
            return i
    return max(range(len(dist)), key=lambda i: dist[i])
