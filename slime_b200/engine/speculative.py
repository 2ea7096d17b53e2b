"""Speculative decoding with the model's own draft head (multi-token prediction, EAGLE-style chain).

One round per engine step for every decoding request, whose known tokens occupy positions ``0 .. L-1`` (the last one
sampled but not yet fed to the model):

1. *draft*: the draft head (one extra transformer layer fed the trunk's residual stream at position p and the embedding
   of token p + 1) already guessed token L when the previous round (or the prefill) ended; ``k - 1`` further single-token
   passes, each fed the head's own stream and its previous guess, extend that to ``k`` guesses ``d_1 .. d_k``;
2. *verify*: one extend pass of the trunk over ``[token L-1, d_1 .. d_k]`` gives the logits of positions ``L .. L+k``;
3. *accept*: every row is sampled with the request's ordinary sampler (same seed, same output position as a
   non-speculative step would use); row ``i + 1`` is valid only if the sample of row ``i`` equals ``d_{i+1}``, so the
   request keeps the samples up to and including the first one that differs. Every kept token is therefore a draw from
   the target distribution given the true prefix (the draft only decides how many rows can be used), log-probs, kept
   top-p sets and routed experts are the trunk's own, and with the counter-based sampler the token sequence is the one
   non-speculative decoding produces;
4. *refresh*: the draft head runs over the accepted positions with the trunk's streams (overwriting what step 1 wrote
   into its cache slab from guessed inputs) and its last row is the next round's first guess.

Cache positions written for rejected guesses are overwritten by the next round, pages are indexed for prefix reuse only
up to the accepted length, and the draft head's keys live in an extra slab of the same pages, so a prefix hit restores
both. The round is driven from the host (accept lengths decide the next inputs), without decode slots or CUDA graphs.

Same role as ``--sglang-speculative-algorithm EAGLE --sglang-speculative-num-steps k --sglang-speculative-eagle-topk 1
--sglang-speculative-num-draft-tokens k+1`` in the reference's MTP recipes (scripts/run-mimo-7B-rl-eagle.sh,
scripts/run-glm4.5-355B-A32B.sh) and the ``spec_*`` counters of ``meta_info`` (slime/utils/types.py:60-90).
"""

from __future__ import annotations

import time

import torch

from slime_b200 import ops
from slime_b200.engine.kv_cache import OutOfPages
from slime_b200.engine.request import Request

ALGORITHMS = ("EAGLE", "EAGLE3", "NEXTN", "MTP")


class SpeculativeDecoder:
    def __init__(self, engine):
        a = engine.args
        if str(a.speculative_algorithm).upper() not in ALGORITHMS:
            raise ValueError(f"unknown speculative algorithm {a.speculative_algorithm!r} (one of {ALGORITHMS})")
        if a.speculative_eagle_topk != 1:
            raise NotImplementedError("draft trees are not built: speculative_eagle_topk must be 1 (a chain of guesses)")
        if a.speculative_draft_model_path:
            raise NotImplementedError("a separate draft model is not supported: the draft head is the checkpoint's own")
        if not engine.weights.draft:
            raise ValueError("speculative decoding needs a model with a draft head (mtp_num_layers >= 1)")
        if engine.runner.has_gdn:
            raise NotImplementedError("speculative decoding over recurrent (delta-net) layers would need state rollback")
        self.eng = engine
        self.k = max(1, int(a.speculative_num_steps))
        if a.speculative_num_draft_tokens not in (None, self.k + 1):
            raise ValueError(f"with a chain of {self.k} guesses the verify pass has {self.k + 1} rows "
                             f"(speculative_num_draft_tokens={a.speculative_num_draft_tokens})")  # fmt: skip

    # ------------------------------------------------------------------ inputs of one packed extend pass
    def _pack(self, spans):
        """``spans``: (request, first position, rows). Device inputs of an extend pass over those positions (new rows
        attend to everything cached before them plus themselves)."""
        eng = self.eng
        pos, slots, cu_q, cu_k, gather, max_q, max_k = [], [], [0], [0], [], 0, 0
        for r, s, n in spans:
            pos += [p + r.rope_delta for p in range(s, s + n)]  # (a request with images rotates by index + offset)
            slots += eng._slots(r, s, s + n)
            cu_q.append(cu_q[-1] + n)
            cu_k.append(cu_k[-1] + s + n)
            gather += eng._slots(r, 0, s + n)
            max_q, max_k = max(max_q, n), max(max_k, s + n)
        t = eng._to_dev
        return t(pos), t(slots), t(cu_q), t(gather, torch.long), t(cu_k), max_q, max_k

    # ------------------------------------------------------------------------------------ prefill hook
    def after_prefill(self, batch, dev_in, cu_q, max_q, max_k, fresh):
        """The draft head over the chunk the trunk just computed (same rows, same cache slots). ``batch``: (request,
        rows) pairs of the pass, with ``num_computed`` already advanced. A request whose prompt is complete gets its first
        guess."""
        eng, run = self.eng, self.eng.runner
        _, pos, slots, cu, gather, cu_k = dev_in
        nxt, last_rows, owners = [], [], []
        for (r, n), a in zip(batch, cu_q[:-1]):
            e = r.num_computed
            ids = r.ctx_ids + r.output_ids[len(r.ctx_ids) - len(r.input_ids):]  # the sampled first token follows the context
            seg = ids[e - n + 1 : e + 1]
            nxt += seg + [0] * (n - len(seg))
            if e == len(r.ctx_ids) and not r.finished() and len(seg) == n:
                last_rows.append(a + n - 1)
                owners.append(r)
        normed, stream = run.draft_extend(0, run.last_hidden, eng._to_dev(nxt), pos, slots, cu, gather, cu_k, max_q, max_k, fresh)
        if owners:
            rows = eng._to_dev(last_rows, torch.long)
            guess = run.logits_of(normed.index_select(0, rows)).argmax(-1).tolist()
            for r, g, row in zip(owners, guess, last_rows):
                r.spec_draft, r.spec_hidden = [int(g)], stream[row]

    # ------------------------------------------------------------------------------------ one round
    def decode_round(self) -> list[Request]:
        eng, run = self.eng, self.eng.runner
        ps = eng.page_size
        # how many guesses each request can use: the length limit and the context window bound the rows
        plan = []
        for r in list(eng.running):
            L = r.seq_len
            room = min(r.sampling.max_new_tokens - len(r.output_ids), eng.max_context - L)
            kr = max(0, min(self.k, room - 1))
            need = -(-(L + kr) // ps) - len(r.pages)
            while need > 0 and r in eng.running:
                try:
                    r.pages += eng.kv.allocator.alloc(need)
                    need = 0
                except OutOfPages:  # the youngest request gives its pages back and is prefilled again later
                    eng._retract(max(eng.running, key=lambda x: x.arrival))
            plan.append((r, L, kr))
        plan = [(r, L, kr) for r, L, kr in plan if r in eng.running]
        if not plan:
            return []
        # 1. chain of guesses
        for j in range(1, self.k):
            live = [(r, L, kr) for r, L, kr in plan if kr > j and len(r.spec_draft) == j]
            if not live:
                continue
            pos, slots, cu, gather, cu_k, mq, mk = self._pack([(r, L - 2 + j, 1) for r, L, _ in live])
            hidden = torch.stack([r.spec_hidden for r, _, _ in live])
            nxt = eng._to_dev([r.spec_draft[-1] for r, _, _ in live])
            normed, stream = run.draft_extend(0, hidden, nxt, pos, slots, cu, gather, cu_k, mq, mk, False)
            guess = run.logits_of(normed).argmax(-1).tolist()
            for i, (r, _, _) in enumerate(live):
                r.spec_draft.append(int(guess[i]))
                r.spec_hidden = stream[i]
        # 2. verify
        spans, ids, row_req, row_idx = [], [], [], []
        for r, L, kr in plan:
            d = (r.spec_draft or [])[:kr]
            kr = len(d)
            spans.append((r, L - 1, kr + 1))
            ids += [r.output_ids[-1]] + d
            row_req += [r] * (kr + 1)
            row_idx += list(range(kr + 1))
        pos, slots, cu, gather, cu_k, mq, mk = self._pack(spans)
        logits = run.prefill(eng._to_dev(ids), pos, slots, cu, gather, cu_k, mq, mk, None, False)
        hidden = run.last_hidden
        routed = run.take_routed()
        eng.stats["decode_steps"] += 1
        # 3. sample every row as an ordinary decode step at its output position would
        dev = logits.device
        f = lambda xs, dt: torch.tensor(xs, dtype=dt, device=dev)  # noqa: E731
        sp = [r.sampling for r in row_req]
        filtered = any(s.top_k > 0 or s.top_p < 1.0 or s.min_p > 0 for s in sp)
        cap = 4096 if filtered and any(s.return_top_p_token_ids for s in sp) else 0
        tok, lp, kept_ids, kept_cnt = ops.sample(
            logits, f([s.temperature for s in sp], torch.float32), f([max(s.top_k, 0) for s in sp], torch.int32) if filtered else None,
            f([s.top_p for s in sp], torch.float32) if filtered else None, f([s.min_p for s in sp], torch.float32) if filtered else None,
            f([r.seed for r in row_req], torch.int64), f([len(r.output_ids) + i for r, i in zip(row_req, row_idx)], torch.int32), cap)  # fmt: skip
        eng.stats["d2h_bytes"] += 8 * len(row_req)
        tok, lp = tok.tolist(), lp.tolist()
        kept_ids = kept_ids.cpu() if kept_ids is not None else None
        kept_cnt = kept_cnt.tolist() if kept_cnt is not None else None
        routed = routed.cpu() if routed is not None else None
        # 4. accept, emit, and collect the rows the draft head is refreshed on
        finished, refresh, a0 = [], [], 0
        for (r, s0, n_rows), d in zip(spans, [(r.spec_draft or [])[: n - 1] for r, _, n in spans]):  # s0: position of row 0
            accepted = 0
            while accepted < len(d) and tok[a0 + accepted] == d[accepted]:
                accepted += 1
            meta = r.extra_meta
            meta["spec_verify_ct"] = meta.get("spec_verify_ct", 0) + 1
            meta["spec_draft_token_num"] = meta.get("spec_draft_token_num", 0) + len(d)
            emitted = 0
            for i in range(accepted + 1):
                if kept_cnt is None and r.sampling.return_top_p_token_ids:
                    r.kept_offsets.append(len(r.kept_ids))  # unfiltered row: the whole vocabulary was kept
                else:
                    eng._record_kept(r, kept_ids, kept_cnt, a0 + i)
                emitted += 1
                if self._emit(r, tok[a0 + i], lp[a0 + i]):
                    break
            meta["spec_accept_token_num"] = meta.get("spec_accept_token_num", 0) + max(emitted - 1, 0)
            eng.stats["decode_tokens"] += emitted
            if r.return_routed_experts and routed is not None:
                r.routed_experts.append(routed[a0 : a0 + emitted])
            r.num_computed = s0 + emitted  # the trunk's keys of the fed tokens that were kept
            if r.finished():
                finished.append(r)
            else:
                eng._commit_pages(r, None)
                refresh.append((r, s0, emitted, a0))
            a0 += n_rows
        # the next round's first guess: the draft head over the kept positions with the trunk's streams
        if refresh:
            pos, slots, cu, gather, cu_k, mq, mk = self._pack([(r, s, n) for r, s, n, _ in refresh])
            rows = [a + i for _, _, n, a in refresh for i in range(n)]
            nxt = [t for r, _, n, _ in refresh for t in r.output_ids[-n:]]
            normed, stream = run.draft_extend(0, hidden.index_select(0, eng._to_dev(rows, torch.long)), eng._to_dev(nxt), pos, slots, cu,
                                              gather, cu_k, mq, mk, False)  # fmt: skip
            ends, acc = [], 0
            for _, _, n, _ in refresh:
                acc += n
                ends.append(acc - 1)
            guess = run.logits_of(normed.index_select(0, eng._to_dev(ends, torch.long))).argmax(-1).tolist()
            for (r, _, _, _), g, e in zip(refresh, guess, ends):
                r.spec_draft, r.spec_hidden = [int(g)], stream[e]
        return finished

    def _emit(self, r: Request, tok: int, lp: float) -> bool:
        """Append one kept token; True when the request ended with it."""
        eng = self.eng
        r.output_ids.append(int(tok))
        r.output_logprobs.append(float(lp))
        sp, n_out, reason = r.sampling, len(r.output_ids), None
        if n_out >= sp.min_new_tokens:
            if not sp.ignore_eos and tok in eng.eos_ids:
                reason = {"type": "stop", "matched": int(tok)}
            elif sp.stop_token_ids and tok in sp.stop_token_ids:
                reason = {"type": "stop", "matched": int(tok)}
            elif sp.stop and eng.tokenizer is not None:
                tail = eng.tokenizer.decode(r.output_ids[-32:])
                hit = next((s for s in sp.stop if s in tail), None)
                if hit is not None:
                    reason = {"type": "stop", "matched": hit}
        if reason is None and n_out >= sp.max_new_tokens:
            reason = {"type": "length", "length": sp.max_new_tokens}
        if reason is None and r.seq_len >= eng.max_context:
            reason = {"type": "length", "length": n_out}
        r.first_token_time = r.first_token_time or time.time()
        if r.on_token is not None:
            r.on_token(r)
        if reason is not None:
            eng.running.remove(r)
            eng._finish(r, reason)
            return True
        return False
