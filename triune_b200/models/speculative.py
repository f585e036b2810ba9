"""Self-speculative decoding: the Reflex exit drafts, the Cortex exit verifies.

Parity: ``SelfSpeculativeGenerator`` (``triune/model/speculative.py:20-221``): draft ``k_draft`` tokens at
``force_depth=0``, verify them with one ``force_depth=2`` pass, greedy acceptance is an exact token match
(the output equals autoregressive Cortex decoding token for token), sampling uses Leviathan rejection
(accept with min(1, p/q), resample from normalised max(p - q, 0) on rejection), one bonus token per round,
telemetry of proposed / accepted / passes.

Difference: the reference re-runs the whole context for every draft token. Here both exits share one recurrent
cache: layers ``0..reflex`` are common to both depths, so drafting advances a working copy of the lower-layer
states one token at a time (O(1) per token), verification is a single k-token chunk through the full stack from
the committed cache, and a partial acceptance recomputes only the accepted prefix.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn.functional as F


def _clone_cache(cache):
    out = []
    for e in cache:
        if isinstance(e, tuple) and e[0] is not None:
            out.append((e[0].clone(), e[1]))
        else:
            out.append(e)
    return out


class SelfSpeculativeGenerator:
    def __init__(self, model, tokenizer=None, k_draft: int = 3, temperature: float = 0.0, pad_token_id: Optional[int] = None,
                 eos_token_id: Optional[int] = None, draft_depth: int = 0, verify_depth: int = 2):
        # positional order of the reference's constructor (``triune/model/speculative.py``); ``temperature`` is the default
        # of ``generate`` when that call names none
        self.model = model
        self.temperature = float(temperature)
        self.tokenizer = tokenizer
        self.k_draft = max(1, int(k_draft))
        self.draft_depth, self.verify_depth = draft_depth, verify_depth
        self.eos_token_id = eos_token_id if eos_token_id is not None else getattr(tokenizer, "sep_token_id", None)
        self.pad_token_id = pad_token_id if pad_token_id is not None else getattr(tokenizer, "pad_token_id", None)
        self.reset_telemetry()

    def reset_telemetry(self):
        self.telemetry = {"proposed": 0, "accepted": 0, "draft_passes": 0, "verify_passes": 0, "rounds": 0,
                          "generated": 0}

    @property
    def acceptance_rate(self) -> float:
        return self.telemetry["accepted"] / max(1, self.telemetry["proposed"])

    @staticmethod
    def _dist(logits, temperature, top_k):
        lg = logits.float()
        if top_k and top_k > 0:
            kth = torch.topk(lg, min(top_k, lg.shape[-1])).values[..., -1:]
            lg = lg.masked_fill(lg < kth, float("-inf"))
        return F.softmax(lg / max(temperature, 1e-6), dim=-1)

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32, temperature: Optional[float] = None, top_k: int = 0,
                 generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """input_ids [1, T]. Returns [1, T + n] with n <= max_new_tokens.

        Invariant between rounds: ``cache`` holds the full-stack state after every committed token except the
        last one, ``last`` is that token. A round drafts k tokens by feeding ``last`` and then each draft through
        the lower stack, verifies with ONE (k+1)-token chunk [last, d1..dk] through the full stack, and commits
        the accepted prefix plus one verifier token.
        """
        model = self.model
        was_training = model.training
        model.eval()
        dev = input_ids.device
        temperature = self.temperature if temperature is None else float(temperature)
        greedy = temperature <= 0
        cache = model.init_cache(input_ids.shape[0])
        if input_ids.shape[1] > 1:
            _, cache = model(input_ids[:, :-1], force_depth=self.verify_depth, cache=cache, last_token_only=True)
            self.telemetry["verify_passes"] += 1
        last = input_ids[:, -1:]
        out: List[int] = []
        done = False
        while len(out) < max_new_tokens and not done:
            self.telemetry["rounds"] += 1
            k = min(self.k_draft, max_new_tokens - len(out))
            # ---- draft on a working copy (only the lower layers are touched at the draft depth)
            work = _clone_cache(cache)
            drafts, q_dists = [], []
            feed = last
            for _ in range(k):
                rl, work = model(feed, force_depth=self.draft_depth, cache=work, last_token_only=True)
                self.telemetry["draft_passes"] += 1
                if greedy:
                    q, tok = None, rl[:, -1].argmax(-1)
                else:
                    q = self._dist(rl[:, -1], temperature, top_k)
                    tok = torch.multinomial(q, 1, generator=generator).squeeze(-1)
                drafts.append(tok)
                q_dists.append(q)
                feed = tok.view(1, 1)
            self.telemetry["proposed"] += k
            chunk = torch.cat([last] + [t.view(1, 1) for t in drafts], dim=1)  # [1, k+1]
            # ---- verify: logits[:, i] is the verifier's prediction for the token after chunk[:, i]
            v_logits, v_cache = model(chunk, force_depth=self.verify_depth, cache=_clone_cache(cache))
            self.telemetry["verify_passes"] += 1
            accepted, bonus = 0, None
            for i in range(k):
                if greedy:
                    tgt = v_logits[:, i].argmax(-1)
                    if int(tgt) == int(drafts[i]):
                        accepted += 1
                        continue
                    bonus = tgt
                    break
                p = self._dist(v_logits[:, i], temperature, top_k)
                tok = drafts[i]
                ratio = (p[0, tok] / q_dists[i][0, tok].clamp_min(1e-20)).clamp(max=1.0)
                if float(torch.rand((), generator=generator)) <= float(ratio):
                    accepted += 1
                    continue
                resid = (p - q_dists[i]).clamp_min(0)
                resid = resid / resid.sum(-1, keepdim=True).clamp_min(1e-20)
                bonus = torch.multinomial(resid, 1, generator=generator).squeeze(-1)
                break
            if bonus is None:  # every draft accepted: the last verifier position yields a free token
                if greedy:
                    bonus = v_logits[:, k].argmax(-1)
                else:
                    bonus = torch.multinomial(self._dist(v_logits[:, k], temperature, top_k), 1,
                                              generator=generator).squeeze(-1)
            self.telemetry["accepted"] += accepted
            # ---- commit [last, d1..d_accepted]; the verifier token becomes the new `last`
            if accepted == k:
                cache = v_cache
            else:
                _, cache = model(chunk[:, : accepted + 1], force_depth=self.verify_depth, cache=cache,
                                 last_token_only=True)
                self.telemetry["verify_passes"] += 1
            last = bonus.view(1, 1)
            for t in [int(x) for x in drafts[:accepted]] + [int(bonus)]:
                out.append(t)
                if (self.eos_token_id is not None and t == self.eos_token_id) or len(out) >= max_new_tokens:
                    done = True
                    break
        self.telemetry["generated"] += len(out)
        model.train(was_training)
        return torch.cat((input_ids, torch.tensor([out], device=dev, dtype=input_ids.dtype)), dim=1)

    @torch.no_grad()
    def generate_autoregressive(self, input_ids: torch.Tensor, max_new_tokens: int = 32) -> torch.Tensor:
        """Greedy Cortex decoding with the recurrent cache (the parity oracle of the speculative path)."""
        model = self.model
        was = model.training
        model.eval()
        cache = model.init_cache(input_ids.shape[0])
        logits, cache = model(input_ids, force_depth=self.verify_depth, cache=cache, last_token_only=True)
        out = []
        for _ in range(max_new_tokens):
            tok = logits[:, -1].argmax(-1)
            out.append(tok)
            if self.eos_token_id is not None and int(tok) == self.eos_token_id:
                break
            logits, cache = model(tok.view(1, 1), force_depth=self.verify_depth, cache=cache, last_token_only=True)
        model.train(was)
        return torch.cat((input_ids, torch.stack(out, dim=1)), dim=1)
