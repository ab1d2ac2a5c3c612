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


class SpeculativeDecoder:
    """Speculative decoding of one sequence with two models of this runtime: a small draft `Decoder` proposes `k`
    tokens one at a time, the target `Decoder` scores the k + 1 positions in ONE chunked forward over its paged KV
    cache, and the longest accepted prefix plus a correction (or bonus) token is kept.

    Both models keep their KV caches across rounds: a round only computes the positions that are new, and cache
    entries written for rejected proposals are overwritten by the next round (attention never reads past the
    sequence length it is given). With temperature 0 the output equals the target's greedy decode; with a
    temperature the accept/reject rule of `core.speculative_verify` makes it a sample from the target.

    Counterpart of the reference's run_speculative_generation over forward_full
    (crates/skein_runtime/src/distributed/gpu_rank.rs:703,2197), which recomputes the whole sequence per call.
    """

    def __init__(self, target, draft, k: int = 4):
        if target.cfg.vocab_size != draft.cfg.vocab_size:
            raise ValueError("draft and target must share the vocabulary")
        if k < 1:
            raise ValueError("k must be at least 1")
        self.target, self.draft, self.k = target, draft, k

    @staticmethod
    def _chunk(dec, tokens, cached: int, table, all_logits: bool):
        """Forward `tokens` at positions cached.. through `dec` (KV appended); logits of every row or the last."""
        import torch

        from ..models.decoder import BatchInputs
        dev, n = dec.device, len(tokens)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        rows = list(range(n)) if all_logits else [n - 1]
        inp = BatchInputs(token_ids=i32(tokens), positions=i32(list(range(cached, cached + n))), block_table=table,
                          seq_lens=i32([cached + n]), is_prefill=True, seq_of_token=i32([0] * n), q_start=i32([0]),
                          q_len=i32([n]), max_q_len=n, logit_rows=torch.tensor(rows, dtype=torch.int64, device=dev))
        _, lg = dec.forward(inp)
        return lg.float()

    def generate(self, prompt, max_new_tokens: int, temperature: float = 0.0, seed: int = 0):
        """Returns (generated tokens, stats) with stats = proposed / accepted / target_steps."""
        import torch
        tgt, drf, k = self.target, self.draft, self.k
        V = tgt.cfg.vocab_size
        total = len(prompt) + max_new_tokens + k + 1
        n_blocks = (total + tgt.page_size - 1) // tgt.page_size
        if n_blocks + 1 > min(tgt.num_pages, drf.num_pages) or total > min(tgt.max_pos, drf.max_pos):
            raise ValueError("sequence does not fit the KV pools or the position limit")
        table_t = torch.arange(1, n_blocks + 1, dtype=torch.int32, device=tgt.device).view(1, -1)
        table_d = torch.arange(1, n_blocks + 1, dtype=torch.int32, device=drf.device).view(1, -1)
        rng = random.Random(seed)
        greedy = temperature <= 0.0

        def probs(lg_row):
            if greedy:
                return None
            return torch.softmax(lg_row[:V] / temperature, dim=-1)

        def pick(lg_row, p):
            if greedy:
                return int(torch.argmax(lg_row[:V]))
            return core_sample(p.tolist(), rng.random())

        seq = [int(t) for t in prompt]
        out: list[int] = []
        stats = {"proposed": 0, "accepted": 0, "target_steps": 0}
        # the target's first token comes from its prefill; from then on `seq` always ends with a token whose KV
        # neither model has computed yet
        lg = self._chunk(tgt, seq, 0, table_t, all_logits=False)
        stats["target_steps"] += 1
        first = pick(lg[0], probs(lg[0]))
        seq.append(first)
        out.append(first)
        t_len = len(seq) - 1          # tokens whose KV is in the target cache
        d_len = 0                     # ... in the draft cache
        while len(out) < max_new_tokens:
            kk = min(k, max_new_tokens - len(out) - 1)
            # ---- draft: catch up on what it has not seen, then propose kk tokens ----
            draft_tokens, draft_ps = [], []
            cur = list(seq)
            for _ in range(kk):
                lg = self._chunk(drf, cur[d_len:], d_len, table_d, all_logits=False)
                d_len = len(cur)
                q = probs(lg[0])
                t = pick(lg[0], q)
                draft_tokens.append(t)
                draft_ps.append(q)
                cur.append(t)
            # ---- target: one forward over [last accepted token, proposals...] ----
            lg = self._chunk(tgt, cur[t_len:], t_len, table_t, all_logits=True)     # kk + 1 rows
            stats["target_steps"] += 1
            stats["proposed"] += kk
            if greedy:
                want = torch.argmax(lg[:, :V], dim=-1).tolist()
                n_acc = 0
                while n_acc < kk and draft_tokens[n_acc] == want[n_acc]:
                    n_acc += 1
                accepted, correction = draft_tokens[:n_acc], int(want[n_acc])
            else:
                ps = [probs(lg[i]).tolist() for i in range(kk + 1)]
                accepted, correction = core.speculative_verify(draft_tokens, [q.tolist() for q in draft_ps], ps,
                                                               [rng.random() for _ in range(kk + 1)])
                accepted, correction = list(accepted), int(correction)
            stats["accepted"] += len(accepted)
            new = (accepted + [correction])[: max_new_tokens - len(out)]
            out.extend(new)
            seq.extend(new)
            # the caches hold valid KV for everything before the last token of `seq`
            t_len = len(seq) - 1
            d_len = min(d_len, len(seq) - 1)
        return out, stats
