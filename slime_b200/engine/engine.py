"""Continuous-batching rollout engine (in-process core).

One ``Engine`` owns the weights, the paged KV cache and a scheduler. ``step()`` either admits
waiting requests and runs a (chunked) prefill over their un-cached tokens, or runs one decode
step for every running request; finished requests free their pages (complete pages stay
indexed for prefix reuse). ``generate()`` is the blocking convenience wrapper; the HTTP server
drives ``step()`` from its scheduler thread.

Decode is pipelined: per-slot token / position state lives on the device, so step ``t+1`` is launched
before the host has looked at step ``t``'s tokens. Sampled tokens and log-probs stream back through a
pinned history ring; the host processes them one step late (length-based finishes need no token at all,
EOS / stop-token finishes are detected one step late and the extra token is discarded).

This is the component that replaces the SGLang server process of the reference
(slime/backends/sglang_utils/sglang_engine.py:88-503 is only its HTTP client); the control
surface it must offer is: generate (with logprobs), abort, pause / continue, flush cache,
release / resume memory by tag (weights | kv_cache | cuda_graph), weight update and versioning.
"""

from __future__ import annotations

import heapq
import threading
import time
import uuid

import numpy as np
import torch

from slime_b200 import ops
from slime_b200.engine.kv_cache import OutOfPages, PagedKVCache, _hash_block
from slime_b200.engine.model_runner import EngineWeights, ModelRunner
from slime_b200.engine.request import ReqState, Request, SamplingParams
from slime_b200.engine.server_args import ServerArgs
from slime_b200.models.config import ModelConfig

MEMORY_TAGS = ("weights", "kv_cache", "cuda_graph")


class Engine:
    def __init__(self, cfg: ModelConfig, server_args: ServerArgs | None = None, device=None, tokenizer=None,
                 num_pages: int | None = None, tp_group=None, tp_size: int = 1, tp_rank: int = 0):  # fmt: skip
        self.cfg = cfg
        self.args = server_args or ServerArgs()
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        )
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.tokenizer = tokenizer
        self.eos_ids: set[int] = set()
        if tokenizer is not None and getattr(tokenizer, "eos_token_id", None) is not None:
            self.eos_ids.add(tokenizer.eos_token_id)
        self.weights = EngineWeights(cfg, self.dtype, self.device, tp_size, tp_rank, ep_size=min(self.args.ep_size, tp_size),
                                     quantization=self.args.quantization,
                                     draft_layers=min(cfg.mtp_num_layers or 0, 1) if self.args.speculative_algorithm else 0)
        self.max_context = self.args.context_length or min(cfg.max_position_embeddings, 32768)
        self.page_size = self.args.page_size
        self.max_running = self.args.max_running_requests
        if num_pages is None:
            num_pages = self._pages_from_memory()
        self.num_pages = num_pages
        kv_heads, kv_dim, v_dim = self._kv_geometry()
        self.kv = PagedKVCache(self._num_kv_layers(), kv_heads, kv_dim, num_pages, self.page_size, self.dtype,
                               self.device, enable_prefix_cache=not self.args.disable_radix_cache, v_head_dim=v_dim)  # fmt: skip
        if self.args.enable_hierarchical_cache and not self.args.disable_radix_cache:
            from slime_b200.engine.kv_cache import HostKVTier

            per_page = PagedKVCache.bytes_per_page(self._num_kv_layers(), kv_heads, kv_dim, self.page_size, self.dtype, v_head_dim=v_dim)
            host_pages = (self.args.hicache_size << 30) // per_page if self.args.hicache_size > 0 else int(num_pages * self.args.hicache_ratio)
            self.kv.allocator.host_tier = HostKVTier(self.kv, host_pages)
        self.runner = ModelRunner(cfg, self.weights, self.kv, self.max_running, self.max_context,
                                  use_cuda_graph=not self.args.disable_cuda_graph, tp_group=tp_group)  # fmt: skip
        self.runner._alloc_static()
        self.runner.record_routed = bool(self.args.enable_return_routed_experts) and cfg.num_experts is not None
        self.routed_hist: dict[int, torch.Tensor] = {}  # decode step -> [slots, moe layers * k] int32 on the host
        self.waiting: list[Request] = []
        self.running: list[Request] = []  # decoding (own a slot) until their results are finalised
        self.prefilling: list[Request] = []
        self.paused = False
        self.released: set[str] = set()
        self.lock = threading.RLock()
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "cached_tokens": 0, "steps": 0, "aborted": 0,
                      "h2d_bytes": 0, "d2h_bytes": 0, "decode_steps": 0}  # fmt: skip
        self._init_decode_state()
        if self.args.enable_deterministic_inference:
            ops.set_batch_invariant(True)  # process-wide: an engine process serves one configuration
        self.spec = None  # host-driven speculative rounds instead of the slot-based decode loop
        if self.args.speculative_algorithm:
            from slime_b200.engine.speculative import SpeculativeDecoder

            self.spec = SpeculativeDecoder(self)

    def _kv_geometry(self):
        """(heads, key width, value width) of one cached token: latent attention caches a single vector per token (the
        compressed key/value plus the shared rotary key) and no separate values."""
        c = self.cfg
        if c.multi_latent_attention:
            return 1, c.kv_lora_rank + c.qk_pos_emb_head_dim + (c.index_head_dim if c.index_topk else 0), 0
        return self.weights.hkv, c.head_dim, None

    def _num_kv_layers(self) -> int:
        """Layers that keep keys and values (delta-net layers keep a recurrent state per decode slot instead)."""
        return sum(1 for L in self.weights.layers + self.weights.draft if L["kind"] in ("attention", "mla"))

    # ----------------------------------------------------------------- sizing
    def _pages_from_memory(self) -> int:
        kv_heads, kv_dim, v_dim = self._kv_geometry()
        per_page = PagedKVCache.bytes_per_page(self._num_kv_layers(), kv_heads, kv_dim, self.page_size, self.dtype, v_head_dim=v_dim)
        if self.args.max_total_tokens:
            return max(8, self.args.max_total_tokens // self.page_size)
        if self.device.type != "cuda":
            return 512
        free, total = torch.cuda.mem_get_info(self.device)
        budget = int(total * self.args.mem_fraction_static) - (total - free)
        return max(64, budget // per_page)

    def _init_decode_state(self):
        B = self.max_running
        self.slot_req: list[Request | None] = [None] * B
        self.free_slots = list(range(B))
        heapq.heapify(self.free_slots)
        self.h_pos = np.zeros(B, dtype=np.int64)  # position of the token the next step feeds
        self.h_remaining = np.zeros(B, dtype=np.int64)  # tokens still to sample (length limit)
        self.h_npages = np.zeros(B, dtype=np.int64)
        self.h_inspect = np.zeros(B, dtype=bool)  # slot needs its tokens looked at (EOS, stop ids, stop strings, stream)
        self.ring = int(min(max(self.max_context + 8, 64), 8192))
        pin = self.device.type == "cuda"
        self.tok_hist = torch.zeros(self.ring, B, dtype=torch.int32, pin_memory=pin)
        self.lp_hist = torch.zeros(self.ring, B, dtype=torch.float32, pin_memory=pin)
        self.tok_np, self.lp_np = self.tok_hist.numpy(), self.lp_hist.numpy()
        self.hist_events: list = [None] * self.ring
        # tensor-parallel decode over peer memory has bounded waits; their status word rides along with the tokens
        self.status_hist = torch.zeros(self.ring, dtype=torch.int32, pin_memory=pin) if self.runner._fused_tp is not None else None
        self.status_np = self.status_hist.numpy() if self.status_hist is not None else None
        self.step_no = 0  # decode steps launched so far
        self.processed = 0  # decode steps whose results the host has consumed
        self.kept_hist: dict[int, tuple] = {}
        if 0 in self.kv.allocator.free:  # page 0 is the scratch page idle decode slots write to
            self.kv.allocator.free.remove(0)
            self.kv.allocator.refcnt[0] = 1

    # ------------------------------------------------------------------ intake
    def add_request(self, input_ids, sampling: SamplingParams | dict | None = None, rid: str | None = None, **kw) -> Request:
        sp = sampling if isinstance(sampling, SamplingParams) else SamplingParams.from_dict(sampling)
        req = Request(rid=rid or uuid.uuid4().hex, input_ids=list(input_ids), sampling=sp, **kw)
        # Without an explicit seed the stream is numbered by arrival order: the ranks of a tensor-parallel engine see the
        # same requests in the same order, so they draw the same tokens (a hash of the random request id would differ
        # from process to process).
        self._req_counter = getattr(self, "_req_counter", 0) + 1
        req.seed = sp.sampling_seed if sp.sampling_seed is not None else (self.args.random_seed * 1000003 + self._req_counter) & 0x7FFFFFFFFFFF
        room = self.max_context - len(req.input_ids)
        if room <= 0:
            self._finish(req, {"type": "length", "length": 0})
            return req
        sp.max_new_tokens = max(0, min(sp.max_new_tokens, room))
        req.weight_version = self.weights.version
        with self.lock:
            self.waiting.append(req)
        return req

    # -------------------------------------------------------------- scheduling
    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self.prefilling)

    def num_requests(self) -> int:
        return len(self.waiting) + len(self.running) + len(self.prefilling)

    def step(self) -> list[Request]:
        """Run one engine iteration; returns requests that finished in it."""
        with self.lock:
            if self.paused or "kv_cache" in self.released or "weights" in self.released:
                return []
            self.stats["steps"] += 1
            batch = self._admit()
            if batch:
                return self._run_prefill(batch)
            if self.running:
                return self.spec.decode_round() if self.spec is not None else self._run_decode()
            return []

    def _admit(self) -> list[tuple[Request, int]]:
        """Pick requests (and how many of their tokens) for this step's prefill, within the token budget."""
        budget = self.args.max_prefill_tokens
        batch: list[tuple[Request, int]] = []
        pending_first_hash = set()
        ps = self.page_size
        for req in list(self.prefilling):  # continue chunked prefills first
            todo = len(req.ctx_ids) - req.num_computed
            n = min(todo, budget, self.args.chunked_prefill_size)
            if n <= 0:
                break
            batch.append((req, n))
            budget -= n
        still_waiting = []
        admitted = 0
        for req in self.waiting:
            if budget <= 0 or len(self.running) + len(self.prefilling) + admitted >= self.max_running:
                still_waiting.append(req)
                continue
            if req.sampling.max_new_tokens == 0 and req.logprob_start_len < 0:
                self._finish(req, {"type": "length", "length": 0})
                continue
            ctx = req.input_ids + req.output_ids  # a retracted request re-enters with what it generated so far
            req.ctx_ids = ctx
            # siblings of a prompt being prefilled right now wait one step and then hit the prefix cache
            first = _hash_block(b"", ctx[:ps]) if len(ctx) > ps else None
            if first is not None and first in pending_first_hash:
                still_waiting.append(req)
                continue
            # input log-probs and routed experts need every position computed
            # (a recurrent layer's state at a page boundary is not kept, so hybrid models do not reuse prefixes either)
            # (image placeholder tokens look the same for every image: such prompts neither reuse nor offer prefixes)
            want_cache = (req.logprob_start_len < 0 and not (req.return_routed_experts and self.runner.record_routed)
                          and not self.runner.has_gdn and req.mm is None)  # fmt: skip
            pages, chain = self.kv.allocator.match_prefix(ctx) if want_cache else ([], b"")
            cached = len(pages) * ps
            total_pages = -(-(len(ctx) + 1) // ps)
            try:
                new_pages = self.kv.allocator.alloc(total_pages - len(pages))
            except OutOfPages:
                self.kv.allocator.release(pages)
                still_waiting.append(req)
                budget = 0
                continue
            req.pages = pages + new_pages
            req.num_cached_tokens = req.num_computed = cached
            req.committed_pages, req.chain_hash = len(pages), chain
            req.first_scheduled = req.first_scheduled or time.time()
            n = min(len(ctx) - cached, budget, self.args.chunked_prefill_size)
            batch.append((req, n))
            admitted += 1
            budget -= n
            self.stats["cached_tokens"] += cached
            if first is not None and cached == 0:
                pending_first_hash.add(first)
        self.waiting = still_waiting
        return batch

    def _slots(self, req: Request, start: int, end: int) -> list[int]:
        ps = self.page_size
        return [req.pages[p // ps] * ps + p % ps for p in range(start, end)]

    def _to_dev(self, x, dt=torch.int32):
        host = torch.tensor(x, dtype=dt)
        self.stats["h2d_bytes"] += host.numel() * host.element_size()
        if self.device.type == "cuda":
            host = host.pin_memory()
        return host.to(self.device, non_blocking=True)

    def _run_prefill(self, batch) -> list[Request]:
        t = self._to_dev
        ids, pos, slots, cu_q, cu_k, gather, last_rows, samplers = [], [], [], [0], [0], [], [], []
        fresh, max_q, max_k = True, 0, 0
        want_all_rows = any(r.logprob_start_len >= 0 for r, _ in batch)
        mrope = self.cfg.mrope_section is not None and any(r.mm is not None for r, _ in batch)
        streams, emb_rows, emb_vecs, emb_deep = [], [], [], []
        for req, n in batch:
            s, e = req.num_computed, req.num_computed + n
            ids += req.ctx_ids[s:e]
            pos += list(range(s, e))
            if req.mm is not None:
                self._prepare_vision(req)
                inside = (req.mm_rows >= s) & (req.mm_rows < e)
                if bool(inside.any()):
                    emb_rows.append(req.mm_rows[inside] - s + cu_q[-1])
                    emb_vecs.append(req.mm_embeds[inside])
                    emb_deep.append([d[inside] for d in req.mm_deepstack])
            if mrope:
                streams.append(self._position_streams(req, s, e))
            slots += self._slots(req, s, e)
            cu_q.append(cu_q[-1] + n)
            cu_k.append(cu_k[-1] + e)
            gather += self._slots(req, 0, e)
            fresh &= s == 0
            max_q, max_k = max(max_q, n), max(max_k, e)
            if e == len(req.ctx_ids):
                last_rows.append(cu_q[-1] - 1)
                samplers.append(req)
            if req.state == ReqState.WAITING:
                req.state = ReqState.RUNNING
                self.prefilling.append(req)
        rows = None if want_all_rows else t(last_rows, torch.long)
        states = [getattr(req, "gdn_state", None) for req, _ in batch] if self.runner.has_gdn else None
        dev_pos = torch.cat(streams, dim=1).to(self.device, torch.int32) if mrope else t(pos)
        dev_in = (t(ids), dev_pos, t(slots), t(cu_q), None if fresh else t(gather, torch.long), t(cu_k))
        embed_rows = None
        if emb_rows:
            deep = [torch.cat([d[k] for d in emb_deep]) for k in range(len(emb_deep[0]))]
            embed_rows = (torch.cat(emb_rows).to(self.device), torch.cat(emb_vecs), deep)
        logits = self.runner.prefill(*dev_in, max_q, max_k, rows, fresh, gdn_states=states, embed_rows=embed_rows)
        if self.runner.has_gdn:
            for (req, _), st in zip(batch, self.runner.last_gdn_states):
                req.gdn_state = st
        self.stats["prefill_tokens"] += len(ids)
        routed = self.runner.take_routed()
        if routed is not None:
            routed = routed.cpu()
            for (req, n), a in zip(batch, cu_q[:-1]):
                if req.return_routed_experts:
                    req.routed_experts.append(routed[a : a + n])
        if want_all_rows:
            self._record_input_logprobs(batch, logits, cu_q)
            logits = logits.index_select(0, t(last_rows, torch.long))
        for req, n in batch:
            req.num_computed += n
            self._commit_pages(req, req.ctx_ids)
        finished = []
        if samplers:
            toks, lps, kept_ids, kept_cnt = self._sample_rows(logits, samplers)
            for i, req in enumerate(samplers):
                self.prefilling.remove(req)
                if req.sampling.max_new_tokens == 0:
                    self._finish(req, {"type": "length", "length": 0})
                    finished.append(req)
                    continue
                req.first_token_time = req.first_token_time or time.time()
                self._record_kept(req, kept_ids, kept_cnt, i)
                if self._append_token(req, toks[i], lps[i]):
                    finished.append(req)
                elif req.prefill_only:
                    req.kv_export = self.export_kv(req)
                    self._finish(req, {"type": "prefill_done"})
                    finished.append(req)
                else:
                    self._start_decoding(req)
        if self.spec is not None:
            self.spec.after_prefill(batch, dev_in, cu_q, max_q, max_k, fresh)
        return finished

    # ------------------------------------------------------------------------- vision inputs
    def _prepare_vision(self, req: Request):
        """First pass of a request with images: run the encoder once, locate the placeholder tokens, lay out the three
        position streams of the prompt. (``image_data`` of ``/generate``: slime/rollout/sglang_rollout.py:158-203 and
        examples/geo3k_vlm_multi_turn/rollout.py:192-209 in the reference send processor-expanded ``input_ids`` plus the
        images.) ``image_embeds`` / ``video_embeds`` (with ``*_deepstack_embeds`` where the encoder has such outputs) in
        place of pixel values skip the encoder: the precomputed-embedding path of engines that split encoder and language
        model."""
        if req.mm_embeds is not None:
            return
        from slime_b200.models.vision import mrope_position_ids

        cfg, mm = self.cfg, req.mm
        ids = torch.tensor(req.input_ids)
        rows, vecs, deep = [], [], []
        n_deep = len((cfg.vision or {}).get("deepstack_visual_indexes") or [])
        for kind, grids, tok in (("image", mm.get("image_grid_thw"), cfg.image_token_id),
                                 ("video", mm.get("video_grid_thw"), cfg.video_token_id)):  # fmt: skip
            values = mm.get("pixel_values" if kind == "image" else "pixel_values_videos")
            ready = mm.get(f"{kind}_embeds")  # encoder outputs computed elsewhere (an encoder-only worker, a cache)
            if values is None and ready is None:
                continue
            where = (ids == tok).nonzero(as_tuple=False).flatten()
            if ready is not None:
                dev, dt = self.runner.device, self.weights.dtype
                out = torch.as_tensor(ready).to(dev, dt)
                extras = [torch.as_tensor(x).to(dev, dt) for x in (mm.get(f"{kind}_deepstack_embeds") or [])]
                if len(extras) != n_deep or any(x.shape != out.shape for x in extras):
                    raise ValueError(f"{kind}_embeds of this model come with {n_deep} same-shaped {kind}_deepstack_embeds")
            else:
                if self.weights.vision is None:
                    raise ValueError("this model has no image encoder")
                out, extras = self.runner.encode_images(torch.as_tensor(values), torch.as_tensor(grids))
            if where.numel() != out.shape[0]:
                raise ValueError(f"{where.numel()} placeholder tokens for {out.shape[0]} encoder vectors")
            rows.append(where)
            vecs.append(out)
            deep.append(extras)
        order = torch.cat(rows).argsort()
        dev_order = order.to(vecs[0].device)
        req.mm_rows, req.mm_embeds = torch.cat(rows)[order], torch.cat(vecs)[dev_order]
        req.mm_deepstack = [torch.cat([d[k] for d in deep])[dev_order] for k in range(len(deep[0]))]
        if cfg.mrope_section:
            merge = (cfg.vision or {}).get("spatial_merge_size", 2)
            g = lambda k: None if mm.get(k) is None else torch.as_tensor(mm[k])  # noqa: E731
            streams, delta = mrope_position_ids(ids, [0, ids.numel()], g("image_grid_thw"), g("video_grid_thw"),
                                                image_token_id=cfg.image_token_id, video_token_id=cfg.video_token_id,
                                                spatial_merge_size=merge)  # fmt: skip
            req.mm_positions, req.rope_delta = streams, int(delta[0])

    def _position_streams(self, req: Request, s: int, e: int) -> torch.Tensor:
        """[3, e - s] rotary positions of context tokens [s, e): the prompt's streams, then index + offset."""
        n_in = len(req.input_ids)
        tail = torch.arange(max(s, n_in), max(e, s, n_in)).expand(3, -1) + req.rope_delta
        if req.mm_positions is None:
            return torch.arange(s, e).expand(3, -1)
        if s >= n_in:
            return tail
        return torch.cat([req.mm_positions[:, s : min(e, n_in)], tail], dim=1)

    # ------------------------------------------------------ prefill / decode disaggregation
    def export_kv(self, req: Request):
        """``(k, v)``, each ``[layers, tokens, kv heads, head dim]``: the cached keys and values of the request's computed
        tokens, copied out of the paged cache (the pages can be released afterwards)."""
        if self.runner.has_gdn:
            raise NotImplementedError("prefill / decode disaggregation does not carry the recurrent state of delta-net layers")
        slots = torch.tensor(self._slots(req, 0, req.num_computed), dtype=torch.long, device=self.device)
        k = torch.stack([kl.index_select(0, slots) for kl in self.kv.k])
        v = torch.stack([vl.index_select(0, slots) for vl in self.kv.v])
        return k, v

    def import_request(self, input_ids, first_token: int, first_logprob: float, kv, sampling: SamplingParams | dict | None = None,
                       rid: str | None = None, **kw) -> Request:  # fmt: skip
        """Decode side of a disaggregated pair: adopt a prompt whose prefill ran on another engine. ``kv`` is what
        ``export_kv`` returned there (any device); it is written into freshly allocated pages and the request starts
        decoding from ``first_token`` without a prefill pass here. Same role as the prefill -> decode KV hand-over of
        the reference's PD-disaggregated rollout servers (slime/ray/rollout.py:46-219, worker types prefill / decode)."""
        if self.spec is not None:
            raise NotImplementedError("a speculating engine cannot adopt a prompt: the draft head's keys are not part of the hand-over")
        sp = sampling if isinstance(sampling, SamplingParams) else SamplingParams.from_dict(sampling)
        req = Request(rid=rid or uuid.uuid4().hex, input_ids=list(input_ids), sampling=sp, **kw)
        self._req_counter = getattr(self, "_req_counter", 0) + 1
        req.seed = sp.sampling_seed if sp.sampling_seed is not None else (self.args.random_seed * 1000003 + self._req_counter) & 0x7FFFFFFFFFFF
        n = len(req.input_ids)
        k, v = kv
        if k.shape[1] != n or k.shape[0] != len(self.kv.k) or tuple(k.shape[2:]) != tuple(self.kv.k[0].shape[1:]):
            raise ValueError(f"KV of shape {tuple(k.shape)} does not fit {n} tokens of this engine's cache "
                             f"[{len(self.kv.k)}, *, {tuple(self.kv.k[0].shape[1:])}]")  # fmt: skip
        sp.max_new_tokens = max(0, min(sp.max_new_tokens, self.max_context - n))
        req.weight_version = self.weights.version
        with self.lock:
            req.pages = self.kv.allocator.alloc(-(-(n + 1) // self.page_size))
            slots = torch.tensor(self._slots(req, 0, n), dtype=torch.long, device=self.device)
            for li in range(len(self.kv.k)):
                self.kv.k[li].index_copy_(0, slots, k[li].to(self.device, self.kv.k[li].dtype))
                self.kv.v[li].index_copy_(0, slots, v[li].to(self.device, self.kv.v[li].dtype))
            req.num_computed = n
            req.ctx_ids = list(req.input_ids)
            req.state = ReqState.RUNNING
            req.first_scheduled = req.first_token_time = time.time()
            self._commit_pages(req, req.ctx_ids)
            self.stats["imported_tokens"] = self.stats.get("imported_tokens", 0) + n
            if not self._append_token(req, int(first_token), float(first_logprob)):
                self._start_decoding(req)
        return req

    def _record_input_logprobs(self, batch, logits, cu_q):
        lsm = torch.log_softmax(logits.float(), -1)
        for (req, n), a, b in zip(batch, cu_q[:-1], cu_q[1:]):
            if req.logprob_start_len < 0:
                continue
            s = req.num_computed
            nxt = torch.tensor(req.ctx_ids[s + 1 : s + n + 1], device=logits.device, dtype=torch.long)
            vals = lsm[a : a + nxt.numel()].gather(-1, nxt[:, None]).squeeze(-1).tolist()
            if req.input_logprobs is None:
                req.input_logprobs = [None]  # the first token has no conditional probability
            req.input_logprobs += vals

    def _sample_rows(self, logits, reqs):
        dev = logits.device
        n = len(reqs)
        f = lambda xs, dt: torch.tensor(xs, dtype=dt, device=dev)  # noqa: E731
        temp = f([r.sampling.temperature for r in reqs], torch.float32)
        filtered = any(r.sampling.top_k > 0 or r.sampling.top_p < 1.0 or r.sampling.min_p > 0 for r in reqs)
        cap = 4096 if any(r.sampling.return_top_p_token_ids for r in reqs) and filtered else 0
        tk = f([max(r.sampling.top_k, 0) for r in reqs], torch.int32) if filtered else None
        tp = f([r.sampling.top_p for r in reqs], torch.float32) if filtered else None
        mp = f([r.sampling.min_p for r in reqs], torch.float32) if filtered else None
        seeds = f([r.seed for r in reqs], torch.int64)
        pos = f([len(r.output_ids) for r in reqs], torch.int32)
        tok, lp, kept_ids, kept_cnt = ops.sample(logits[:n], temp, tk, tp, mp, seeds, pos, cap)
        self.stats["d2h_bytes"] += 8 * n
        return tok.tolist(), lp.tolist(), (kept_ids.cpu() if kept_ids is not None else None), (
            kept_cnt.tolist() if kept_cnt is not None else None
        )

    # ------------------------------------------------------------------ decode slots
    def _needs_inspection(self, r: Request) -> bool:
        sp = r.sampling
        return bool((not sp.ignore_eos and self.eos_ids) or sp.stop_token_ids or sp.stop or r.on_token is not None)

    def _start_decoding(self, r: Request):
        """Give the request a decode slot; its first input token and position reach the device with the next upload."""
        if self.spec is not None:  # speculative rounds are driven from the request's own lists: no slot, no device state
            r.slot, r.end_step = None, None
            self.running.append(r)
            return
        b = heapq.heappop(self.free_slots)
        h = self.runner.host
        L = r.seq_len
        r.slot, r.decode_from_step, r.harvested = b, self.step_no, self.step_no
        self.slot_req[b] = r
        if self.runner.rope_delta is not None:
            self.runner.rope_delta[b] = r.rope_delta
        if self.runner.has_gdn:
            self.runner.load_gdn_state(b, r.gdn_state)
            r.gdn_state = None
        h["active"][b], h["init_mask"][b] = 1, 1
        h["init_ids"][b], h["init_pos"][b], h["init_out_pos"][b] = r.output_ids[-1], L - 1, len(r.output_ids)
        h["top_k"][b], h["temperature"][b] = max(r.sampling.top_k, 0), r.sampling.temperature
        h["top_p"][b], h["min_p"][b], h["seeds"][b] = r.sampling.top_p, r.sampling.min_p, r.seed
        bt = h["block_table"][b]
        bt[:] = 0
        bt[: len(r.pages)] = r.pages
        self.h_pos[b], self.h_npages[b] = L - 1, len(r.pages)
        self.h_remaining[b] = r.sampling.max_new_tokens - len(r.output_ids)
        self.h_inspect[b] = self._needs_inspection(r)
        r.end_step = None  # decode step index (exclusive) up to which this request's tokens count
        self.running.append(r)

    def _deactivate(self, b: int):
        self.runner.host["active"][b] = 0
        self.runner.host["block_table"][b, :] = 0

    def _release_slot(self, r: Request):
        if r.slot is None:  # a request of the speculative loop
            if r in self.running:
                self.running.remove(r)
            return
        b = r.slot
        self._deactivate(b)
        self.slot_req[b] = None
        self.h_inspect[b] = False
        heapq.heappush(self.free_slots, b)
        r.slot = None
        if r in self.running:
            self.running.remove(r)

    def _run_decode(self) -> list[Request]:
        h = self.runner.host
        ps = self.page_size
        act = h["active"][: self.max_running].astype(bool)
        finished: list[Request] = []
        if not act.any():
            return self._drain()
        # a slot whose next token starts a new page needs that page before the launch; when the cache is
        # full the youngest request is retracted (its KV is rebuilt when it is re-admitted)
        need = np.nonzero(act & (self.h_pos // ps >= self.h_npages))[0]
        for b in need:
            r = self.slot_req[b]
            if r is None or not h["active"][b]:
                continue
            try:
                r.pages += self.kv.allocator.alloc(1)
            except OutOfPages:
                victim = max((x for x in self.running if x.slot is not None and h["active"][x.slot]), key=lambda x: x.arrival)
                self._sync_results()
                self._retract(victim)
                if victim is r:
                    continue
                r.pages += self.kv.allocator.alloc(1)
            h["block_table"][b, len(r.pages) - 1] = r.pages[-1]
            self.h_npages[b] = len(r.pages)
        act = h["active"][: self.max_running].astype(bool)
        if not act.any():
            return self._drain()
        n = int(np.nonzero(act)[0][-1]) + 1
        filtered = bool((h["top_k"][:n][act[:n]] > 0).any() or (h["top_p"][:n][act[:n]] < 1.0).any() or (h["min_p"][:n][act[:n]] > 0).any())
        cap = 4096 if filtered and any(r.sampling.return_top_p_token_ids for r in self.running) else 0
        self.stats["h2d_bytes"] += self.runner.upload_static()
        tok, lp, kept_ids, kept_cnt = self.runner.decode(n, filtered, cap)
        # results stream back into the pinned history ring; an event marks their arrival
        slot = self.step_no % self.ring
        self.tok_hist[slot, :n].copy_(tok[:n], non_blocking=True)
        self.lp_hist[slot, :n].copy_(lp[:n], non_blocking=True)
        if self.status_hist is not None:
            from slime_b200.ops import _lib

            self.status_hist[slot : slot + 1].copy_(_lib.status_word(self.device), non_blocking=True)
        if self.runner.last_routed is not None and any(r.return_routed_experts for r in self.running):
            host = torch.empty(self.runner.last_routed[:n].shape, dtype=torch.int32, pin_memory=self.device.type == "cuda")
            host.copy_(self.runner.last_routed[:n], non_blocking=True)  # ordered before the step's event
            self.routed_hist[self.step_no] = host
            self.stats["d2h_bytes"] += host.numel() * 4
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.hist_events[slot] = ev
        if cap:
            self.kept_hist[self.step_no] = (kept_ids[:n].cpu(), kept_cnt[:n].cpu())
        self.stats["d2h_bytes"] += 8 * n
        self.stats["decode_tokens"] += int(act.sum())
        self.stats["decode_steps"] += 1
        self.step_no += 1
        # host mirrors advance without looking at the tokens
        self.h_pos[act] += 1
        self.h_remaining[act] -= 1
        done = np.nonzero(act & (self.h_remaining <= 0))[0]
        for b in done:
            r = self.slot_req[b]
            if r.end_step is None:
                r.end_step, r.end_reason = self.step_no, {"type": "length", "length": r.sampling.max_new_tokens}
            self._deactivate(b)
        # consume the previous step's results while this one runs
        finished += self._process_until(self.step_no - 1)
        if (self.routed_hist or self.kept_hist) and self.step_no % 64 == 0:  # drop per-step records every reader is past
            low = min((r.harvested for r in self.running), default=self.step_no)
            for hist in (self.routed_hist, self.kept_hist):
                for s_ in [s_ for s_ in hist if s_ < low]:
                    del hist[s_]
        if self.step_no - min((r.harvested for r in self.running), default=self.step_no) > self.ring // 2:
            self._sync_results()
            for r in self.running:
                self._harvest(r, self.processed)
        return finished

    def _drain(self) -> list[Request]:
        """No active slot left: consume every outstanding result."""
        return self._process_until(self.step_no)

    def _sync_results(self):
        self._process_until(self.step_no, finalize=False)

    def _process_until(self, upto: int, finalize: bool = True) -> list[Request]:
        """Consume decode results of steps [processed, upto): token inspection (EOS / stop) for the slots that
        need it, then finalise requests whose end step has been consumed."""
        finished = []
        while self.processed < upto:
            s = self.processed
            slot = s % self.ring
            ev = self.hist_events[slot]
            if ev is not None:
                ev.synchronize()
            if self.status_np is not None and self.status_np[slot] != 0:
                from slime_b200.ops import _lib

                code = int(self.status_np[slot])
                _lib.status_word(self.device).zero_()
                raise _lib.KernelWaitExpired(code & 0xFF, code >> 8)  # this step's hidden states were not all written
            if self.h_inspect.any():
                for b in np.nonzero(self.h_inspect)[0]:
                    r = self.slot_req[b]
                    if r is None or r.end_step is not None and s >= r.end_step or s < r.decode_from_step:
                        continue
                    self._inspect_token(r, s, int(self.tok_np[slot, b]))
            self.processed += 1
        if finalize:
            for r in list(self.running):
                if r.end_step is not None and r.end_step <= self.processed:
                    self._harvest(r, r.end_step)
                    self._release_slot(r)
                    self._finish(r, r.end_reason)
                    finished.append(r)
        return finished

    def _inspect_token(self, r: Request, step: int, tok: int):
        """Stop conditions that depend on the token value. ``step`` is the decode step that sampled ``tok``."""
        sp = r.sampling
        n_out = len(r.output_ids) + (step - r.harvested) + 1
        reason = None
        if n_out >= sp.min_new_tokens:
            if not sp.ignore_eos and tok in self.eos_ids:
                reason = {"type": "stop", "matched": tok}
            elif sp.stop_token_ids and tok in sp.stop_token_ids:
                reason = {"type": "stop", "matched": tok}
            elif sp.stop and self.tokenizer is not None:
                self._harvest(r, step + 1)
                tail = self.tokenizer.decode(r.output_ids[-32:])
                for s_ in sp.stop:
                    if s_ in tail:
                        reason = {"type": "stop", "matched": s_}
                        break
        if r.on_token is not None:
            self._harvest(r, step + 1)
            r.on_token(r)
        if reason is not None:
            r.end_step, r.end_reason = step + 1, reason
            if r.slot is not None:
                self._deactivate(r.slot)  # a token sampled after this one is discarded

    def _harvest(self, r: Request, upto: int):
        """Move the request's tokens of decode steps [harvested, upto) from the history ring into its lists."""
        if r.slot is None or upto <= r.harvested:
            return
        b = r.slot
        steps = np.arange(r.harvested, upto) % self.ring
        r.output_ids += self.tok_np[steps, b].tolist()
        r.output_logprobs += self.lp_np[steps, b].tolist()
        if r.sampling.return_top_p_token_ids:
            for s in range(r.harvested, upto):
                kept = self.kept_hist.get(s)
                if kept is None:
                    r.kept_offsets.append(len(r.kept_ids))
                    continue
                c = max(int(kept[1][b]), 0)
                r.kept_ids += kept[0][b, :c].tolist()
                r.kept_offsets.append(len(r.kept_ids))
        if r.return_routed_experts:
            for s in range(r.harvested, upto):
                hist = self.routed_hist.get(s)
                if hist is not None and b < hist.shape[0]:
                    r.routed_experts.append(hist[b : b + 1].clone())
        r.harvested = upto
        r.num_computed = len(r.input_ids) + len(r.output_ids) - 1
        self._commit_pages(r, None)

    def _retract(self, req: Request):
        """Return a decoding request to the queue: tokens generated so far are kept and re-prefilled later."""
        self._harvest(req, self.processed)
        self._release_slot(req)
        req.routed_experts = []  # the re-prefill computes every position again
        req.gdn_state = None
        req.spec_draft, req.spec_hidden = [], None
        self.kv.allocator.release(req.pages)
        req.pages, req.num_computed, req.committed_pages, req.chain_hash = [], 0, 0, b""
        req.state = ReqState.WAITING
        self.waiting.insert(0, req)

    def _commit_pages(self, req: Request, ids):
        """Index every page that became full and whose KV is written (committed tokens only)."""
        if req.mm is not None:
            return
        ps = self.page_size
        while (req.committed_pages + 1) * ps <= req.num_computed and req.committed_pages < len(req.pages):
            ids = ids or (req.input_ids + req.output_ids)
            i = req.committed_pages
            req.chain_hash = self.kv.allocator.commit(req.pages[i], req.chain_hash, ids[i * ps : (i + 1) * ps])
            req.committed_pages += 1

    def _record_kept(self, req, kept_ids, kept_cnt, row):
        if kept_cnt is not None and req.sampling.return_top_p_token_ids:
            c = max(kept_cnt[row], 0)
            req.kept_ids += kept_ids[row, :c].tolist() if kept_ids is not None and c > 0 else []
            req.kept_offsets.append(len(req.kept_ids))

    def _append_token(self, req: Request, tok: int, lp: float) -> bool:
        """First token (sampled from the prefill logits). Returns True when the request is already finished."""
        req.output_ids.append(int(tok))
        req.output_logprobs.append(float(lp))
        sp = req.sampling
        n_out = len(req.output_ids)
        reason = None
        if n_out >= sp.min_new_tokens:
            if not sp.ignore_eos and tok in self.eos_ids:
                reason = {"type": "stop", "matched": int(tok)}
            elif sp.stop_token_ids and tok in sp.stop_token_ids:
                reason = {"type": "stop", "matched": int(tok)}
        if reason is None and n_out >= sp.max_new_tokens:
            reason = {"type": "length", "length": sp.max_new_tokens}
        if req.on_token is not None:
            req.on_token(req)
        if reason is not None:
            self._finish(req, reason)
            return True
        return False

    def _finish(self, req: Request, reason: dict):
        req.finish_reason = reason
        req.state = ReqState.FINISHED
        req.finish_time = time.time()
        if req in self.prefilling:
            self.prefilling.remove(req)
        if req.pages:
            self.kv.allocator.release(req.pages)
            req.pages = []
        if req.done_event is not None:
            req.done_event.set()
        if req.on_token is not None and reason.get("type") == "abort":
            req.on_token(req)

    # ---------------------------------------------------------------- control plane
    def abort(self, rid: str | None = None, abort_all: bool = False) -> int:
        with self.lock:
            victims = [r for r in self.waiting + self.prefilling + self.running if abort_all or r.rid == rid]
            if any(r in self.running for r in victims):
                self._sync_results()
            for r in victims:
                if r in self.waiting:
                    self.waiting.remove(r)
                if r in self.running:
                    self._harvest(r, self.processed if r.end_step is None else min(r.end_step, self.processed))
                    self._release_slot(r)
                self._finish(r, {"type": "abort"})
            self.stats["aborted"] += len(victims)
            return len(victims)

    def pause_generation(self):
        self.paused = True

    def continue_generation(self):
        self.paused = False

    def flush_cache(self) -> bool:
        with self.lock:
            if self.running or self.prefilling:
                return False
            self.kv.allocator.flush()
            return True

    def release_memory_occupation(self, tags=None):
        """Idempotent per tag. Weights are dropped, not backed up: the trainer re-syncs them after every resume."""
        with self.lock:
            for tag in tags or MEMORY_TAGS:
                if tag in self.released:
                    continue
                if tag == "kv_cache":
                    self.abort(abort_all=True)
                    self.kv.release()
                    if self.args.release_hicache and self.kv.allocator.host_tier is not None:
                        self.kv.allocator.host_tier.release()  # the host pool goes too; without the switch it survives
                elif tag == "cuda_graph":
                    self.runner.drop_graphs()
                elif tag == "weights":
                    for t in self.weights.tensors():
                        t.data = torch.empty(0, dtype=t.dtype, device=t.device)
                self.released.add(tag)
            if self.device.type == "cuda":
                torch.cuda.empty_cache()

    def resume_memory_occupation(self, tags=None):
        with self.lock:
            for tag in tags or MEMORY_TAGS:
                if tag not in self.released:
                    continue
                if tag == "kv_cache":
                    self.kv.allocate()
                    if self.kv.allocator.host_tier is not None:
                        self.kv.allocator.host_tier.allocate()
                    if 0 in self.kv.allocator.free:
                        self.kv.allocator.free.remove(0)
                        self.kv.allocator.refcnt[0] = 1
                elif tag == "weights":
                    fresh = EngineWeights(self.cfg, self.dtype, self.device, self.weights.tp, self.weights.rank, ep_size=self.weights.ep,
                                          quantization=self.weights.quantization, draft_layers=self.weights.num_draft_layers)
                    fresh.version = self.weights.version
                    self.weights = fresh
                    self.runner.w = fresh
                    self.runner.drop_graphs()
                self.released.discard(tag)

    def shutdown(self):
        """Release what must be gone before the process group is destroyed. A tensor-parallel engine captures NCCL
        collectives (embedding all-reduce, logits all-gather) in its decode graphs; NCCL does not finish destroying a
        communicator while graphs that recorded its collectives are alive, so ``destroy_process_group`` blocks forever
        unless the graphs are dropped first."""
        import gc

        with self.lock:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.runner.drop_graphs()
            self.runner._fused_tp = None
        gc.collect()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def update_weights(self, named_tensors, version: str | None = None, flush_cache: bool = True):
        with self.lock:
            missing = self.weights.load_weights(named_tensors, version)
            if flush_cache:
                self.kv.allocator.flush()
            return missing

    def get_weight_version(self) -> str:
        return self.weights.version

    def loads(self) -> dict:
        return {"num_running_reqs": len(self.running) + len(self.prefilling), "num_waiting_reqs": len(self.waiting),
                "num_reqs": self.num_requests(), **self.kv.allocator.stats()}  # fmt: skip

    # ------------------------------------------------------------------- blocking API
    def generate(self, prompts: list[list[int]], sampling: list[dict | SamplingParams] | dict | SamplingParams | None = None,
                 **kw) -> list[Request]:
        if not isinstance(sampling, list):
            sampling = [sampling] * len(prompts)
        reqs = [self.add_request(p, SamplingParams.from_dict(s) if isinstance(s, dict) or s is None else s, **kw)
                for p, s in zip(prompts, sampling)]  # fmt: skip
        while any(not r.finished() for r in reqs):
            if not self.has_work():
                break
            self.step()
        return reqs

    def meta_info(self, req: Request) -> dict:
        """The ``meta_info`` dict of a finished (or streaming) request, in the wire format slime consumes."""
        from slime_b200.utils.misc import encode_int32_meta_array

        now = req.finish_time or time.time()
        e2e = now - req.arrival
        decode_time = max(now - (req.first_token_time or now), 1e-9)
        m = {
            "id": req.rid,
            "finish_reason": req.finish_reason,
            "prompt_tokens": len(req.input_ids),
            "completion_tokens": len(req.output_ids),
            "cached_tokens": req.num_cached_tokens,
            "weight_version": req.weight_version,
            "e2e_latency": e2e,
            "queue_time": (req.first_scheduled or now) - req.arrival,
            "decode_throughput": max(len(req.output_ids) - 1, 0) / decode_time,
            "output_token_logprobs": [(lp, t, None) for lp, t in zip(req.output_logprobs, req.output_ids)],
        }
        if req.input_logprobs is not None:
            m["input_token_logprobs"] = [(lp, t, None) for lp, t in zip(req.input_logprobs, req.input_ids)]
        if req.sampling.return_top_p_token_ids and len(req.kept_offsets) > 1:
            m["top_p_token_ids"] = encode_int32_meta_array(req.kept_ids)
            m["top_p_token_offsets"] = encode_int32_meta_array(req.kept_offsets)
        if req.return_routed_experts and req.routed_experts:
            m["routed_experts"] = encode_int32_meta_array(torch.cat(req.routed_experts).reshape(-1))
        m.update(req.extra_meta)
        return m
