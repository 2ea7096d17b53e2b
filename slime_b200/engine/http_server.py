"""HTTP front of the rollout engine, speaking the SGLang-compatible surface the rollout code uses.

Endpoints (callers in the reference: slime/rollout/sglang_rollout.py:152-221,
slime/backends/sglang_utils/sglang_engine.py:239-492, server_control.py:32-67):
  POST /generate (JSON or SSE stream)      GET  /health, /health_generate, /get_model_info
  POST /abort_request {rid|abort_all}      GET  /v1/loads (also /get_load)
  GET|POST /flush_cache                    POST /pause_generation, /continue_generation
  POST /release_memory_occupation, /resume_memory_occupation {tags}
  POST /update_weights_from_tensor, /update_weights_from_disk, /pull_weights
  POST /init_weights_update_group, /destroy_weights_update_group, /update_weights_from_distributed
  GET  /get_weight_version, /weight_version   POST /weights_checker {action}
  POST /post_process_weights               POST /start_profile, /stop_profile
  GET  /server_info, /get_server_info      GET  /metrics (Prometheus text)

The engine core runs on a dedicated scheduler thread (``Engine.step`` in a loop); aiohttp handlers only
enqueue requests and await their completion events, so control endpoints never block on a busy scheduler.
"""

from __future__ import annotations

import asyncio
import base64
import io
import json
import os
import threading
import time

import torch

from slime_b200.engine.engine import MEMORY_TAGS, Engine
from slime_b200.engine.request import SamplingParams


class EngineServer:
    def __init__(self, engine: Engine, host: str = "127.0.0.1", port: int = 30000, tokenizer=None, processor=None):
        self.engine, self.host, self.port = engine, host, port
        self.tokenizer = tokenizer or engine.tokenizer
        self.processor = processor  # multimodal processor of the checkpoint, when it ships one
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._loop: asyncio.AbstractEventLoop | None = None
        self._runner = None
        self._wake = threading.Event()
        self.started_at = time.time()
        self._weights_snapshot = None
        self._update_groups: dict[str, object] = {}
        self.num_generated = 0
        # prefill / decode disaggregation: KV of finished prefill-only requests, waiting for their decode worker
        self.kv_store: dict[str, tuple] = {}
        self.kv_store_ttl = 600.0

    # ------------------------------------------------------------------ scheduler thread
    def _scheduler_loop(self):
        if self.engine.device.type == "cuda":
            torch.cuda.set_device(self.engine.device)
        while not self._stop.is_set():
            if self.engine.has_work() and not self.engine.paused:
                try:
                    self.engine.step()
                except Exception as e:  # noqa: BLE001  surface the failure on every pending request
                    self.engine.abort(abort_all=True)
                    self.last_error = repr(e)
            else:
                self._wake.wait(timeout=0.002)
                self._wake.clear()

    # ---------------------------------------------------------------------------- handlers
    def _vision_inputs(self, image_data, ids, text, video_data=None):
        """``image_data`` (base64 / data URLs / paths, one request) and ``video_data`` (a list of clips, each a list of
        frames given the same way) -> (prompt ids with every placeholder run at its full length, encoder inputs). With
        ``input_ids`` the prompt is taken as sent (already expanded by the caller's processor, or one placeholder per
        image and per frame group of a clip, each group between its own markers); with ``text`` it is tokenised here."""
        from slime_b200.utils.image_processing import ImageProcessor, expand_image_placeholders
        from slime_b200.utils.processing_utils import _load_image

        cfg = self.engine.cfg
        if cfg.vision is None or cfg.image_token_id is None:
            raise ValueError("this model takes no images")
        if video_data and cfg.video_token_id is None:
            raise ValueError("this model takes no videos")
        images = [_load_image(x) for x in (image_data if isinstance(image_data, list) else [image_data])] if image_data else []
        videos = [[_load_image(f) for f in clip] for clip in (video_data or [])]
        own = ImageProcessor.from_vision_config(cfg.vision)
        mm = {}
        if images:
            ip = getattr(self.processor, "image_processor", None)
            out = ip(images=images, return_tensors="pt") if ip is not None else own(images)
            mm.update(pixel_values=out["pixel_values"], image_grid_thw=out["image_grid_thw"])
        if videos:
            vp = getattr(self.processor, "video_processor", None)
            out = vp(videos=videos, return_tensors="pt") if vp is not None else own(videos=videos)
            mm.update(pixel_values_videos=out["pixel_values_videos"], video_grid_thw=out["video_grid_thw"])
        if ids is None:
            if text is None or self.tokenizer is None:
                raise ValueError("input_ids (or text with a tokenizer) required")
            ids = self.tokenizer.encode(text, add_special_tokens=False)
        merge = cfg.vision.get("spatial_merge_size", 2) ** 2
        ids = list(ids)
        if images:
            ids = expand_image_placeholders(ids, cfg.image_token_id, [int(t * h * w) // merge for t, h, w in mm["image_grid_thw"].tolist()])
        if videos:  # one run per frame group
            counts = [int(h * w) // merge for t, h, w in mm["video_grid_thw"].tolist() for _ in range(int(t))]
            ids = expand_image_placeholders(ids, cfg.video_token_id, counts)
        return ids, mm

    async def _generate(self, request):
        from aiohttp import web

        body = await request.json()
        ids = body.get("input_ids")
        mm = None
        if body.get("image_data") or body.get("video_data"):
            try:
                ids, mm = self._vision_inputs(body.get("image_data"), ids, body.get("text"), body.get("video_data"))
            except Exception as e:  # noqa: BLE001  a bad image or a prompt that does not match its images
                return web.json_response({"error": f"vision inputs: {e}"}, status=400)
        if ids is None:
            text = body.get("text")
            if text is None or self.tokenizer is None:
                return web.json_response({"error": "input_ids (or text with a tokenizer) required"}, status=400)
            ids = self.tokenizer.encode(text, add_special_tokens=False)
        batched = bool(ids) and isinstance(ids[0], list)
        prompts = ids if batched else [ids]
        sp = body.get("sampling_params") or {}
        sps = sp if isinstance(sp, list) else [sp] * len(prompts)
        loop = asyncio.get_running_loop()
        stream = bool(body.get("stream"))
        prefill_only = body.get("disaggregation") == "prefill"
        room = body.get("bootstrap_room")
        if room is not None and not batched:
            return await self._generate_imported(body, ids, sps[0], room)
        reqs, events, queues = [], [], []
        for p, s in zip(prompts, sps):
            ev = asyncio.Event()
            q: asyncio.Queue = asyncio.Queue()

            class _Done:  # thread-safe bridge from the scheduler thread to the event loop
                def __init__(self, ev):
                    self.ev = ev

                def set(self):
                    loop.call_soon_threadsafe(self.ev.set)

            def on_token(r, q=q):
                if stream:
                    loop.call_soon_threadsafe(q.put_nowait, len(r.output_ids))

            req = self.engine.add_request(
                p, SamplingParams.from_dict(s), rid=body.get("rid"), return_logprob=bool(body.get("return_logprob", False)),
                logprob_start_len=int(body.get("logprob_start_len", -1) if body.get("return_logprob") else -1),
                return_routed_experts=bool(body.get("return_routed_experts", False)), stream=stream,
                on_token=on_token if stream else None, done_event=_Done(ev), prefill_only=prefill_only, mm=mm,
            )  # fmt: skip
            if req.finished():
                ev.set()
            reqs.append(req)
            events.append(ev)
            queues.append(q)
        self._wake.set()
        if stream and not batched:
            resp = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
            await resp.prepare(request)
            req, ev, q = reqs[0], events[0], queues[0]
            while not ev.is_set():
                try:
                    await asyncio.wait_for(q.get(), timeout=0.05)
                except asyncio.TimeoutError:
                    continue
                await resp.write(f"data: {json.dumps(self._render(req))}\n\n".encode())
            await resp.write(f"data: {json.dumps(self._render(req))}\n\n".encode())
            await resp.write(b"data: [DONE]\n\n")
            return resp
        await asyncio.gather(*[e.wait() for e in events])
        self.num_generated += sum(len(r.output_ids) for r in reqs)
        out = [self._render(r) for r in reqs]
        if prefill_only:
            now = time.time()
            for rid in [k for k, (_, t0) in self.kv_store.items() if now - t0 > self.kv_store_ttl]:
                del self.kv_store[rid]  # a decode worker that never came
            for r, o in zip(reqs, out):
                if r.kv_export is not None:
                    self.kv_store[r.rid] = (r.kv_export, now)
                    r.kv_export = None
                    o["meta_info"]["kv_handle"] = r.rid
        return web.json_response(out if batched else out[0])

    async def _kv_fetch(self, request):
        """Decode worker's pull of a prefilled prompt's KV: 4-byte little-endian header length, a JSON header (shape,
        dtype), then the raw bytes of k and of v. The entry is dropped once served."""
        from aiohttp import web

        entry = self.kv_store.pop(request.match_info["rid"], None)
        if entry is None:
            return web.json_response({"error": "unknown or expired KV handle"}, status=404)
        (k, v), _ = entry
        k, v = k.contiguous().cpu(), v.contiguous().cpu()
        header = json.dumps({"shape": list(k.shape), "dtype": str(k.dtype).replace("torch.", "")}).encode()
        raw = lambda t: t.view(torch.uint8).numpy().tobytes()  # noqa: E731
        return web.Response(body=len(header).to_bytes(4, "little") + header + raw(k) + raw(v), content_type="application/octet-stream")

    async def _generate_imported(self, body, ids, sampling, room):
        """Decode side: pull the KV from the prefill worker named in the request and continue from its first token."""
        import aiohttp
        from aiohttp import web

        host = body["bootstrap_host"]
        limit = float(os.environ.get("SLIME_B200_DISAGG_TRANSFER_TIMEOUT", "600"))  # a stuck transfer ends with 504
        t0 = time.time()
        try:
            async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=limit)) as s, s.get(f"{host}/disagg/kv/{room}") as resp:
                if resp.status != 200:
                    return web.json_response({"error": f"KV {room} not available at {host}"}, status=502)
                blob = await resp.read()
        except asyncio.TimeoutError:
            return web.json_response({"error": f"KV transfer from {host} exceeded {limit:.0f} s"}, status=504)
        transfer_s = max(time.time() - t0, 1e-9)
        n = int.from_bytes(blob[:4], "little")
        header = json.loads(blob[4 : 4 + n])
        dt = getattr(torch, header["dtype"])
        count = 1
        for d in header["shape"]:
            count *= d
        nbytes = count * torch.empty(0, dtype=dt).element_size()
        body_bytes = memoryview(blob)[4 + n :]
        k = torch.frombuffer(bytearray(body_bytes[:nbytes]), dtype=dt).view(header["shape"])
        v = torch.frombuffer(bytearray(body_bytes[nbytes : 2 * nbytes]), dtype=dt).view(header["shape"])
        loop = asyncio.get_running_loop()
        ev = asyncio.Event()

        class _Done:
            def set(self_inner):
                loop.call_soon_threadsafe(ev.set)

        try:
            req = self.engine.import_request(ids, int(body["first_token"]), float(body.get("first_logprob", 0.0)), (k, v),
                                             SamplingParams.from_dict(sampling), rid=body.get("rid"),
                                             return_logprob=bool(body.get("return_logprob", False)), done_event=_Done())  # fmt: skip
        except Exception as e:  # noqa: BLE001 - out of pages, shape mismatch
            return web.json_response({"error": repr(e)}, status=503)
        mb = len(blob) / 1e6
        req.extra_meta.update(pd_transfer_total_mb=mb, pd_transfer_duration=transfer_s, pd_transfer_speed_gb_s=mb / 1e3 / transfer_s,
                              pd_prefill_host=host, pd_prefill_retry_count=0)  # fmt: skip
        if req.finished():
            ev.set()
        self._wake.set()
        await ev.wait()
        self.num_generated += len(req.output_ids)
        return web.json_response(self._render(req))

    # ---------------------------------------------------------------- OpenAI-compatible front end
    async def _run_one(self, ids: list[int], sampling: dict, rid=None):
        """Submit one request and wait for it (shared by the chat and completion endpoints)."""
        loop = asyncio.get_running_loop()
        ev = asyncio.Event()

        class _Done:
            def set(self_inner):
                loop.call_soon_threadsafe(ev.set)

        req = self.engine.add_request(ids, SamplingParams.from_dict(sampling), rid=rid, return_logprob=False, done_event=_Done())
        if req.finished():
            ev.set()
        self._wake.set()
        await ev.wait()
        self.num_generated += len(req.output_ids)
        return req

    @staticmethod
    def _openai_sampling(body: dict) -> dict:
        sp = {"max_new_tokens": int(body.get("max_tokens") or body.get("max_completion_tokens") or 128)}
        for src, dst in (("temperature", "temperature"), ("top_p", "top_p"), ("top_k", "top_k"), ("min_p", "min_p"),
                         ("stop", "stop"), ("seed", "sampling_seed")):  # fmt: skip
            if body.get(src) is not None:
                sp[dst] = body[src]
        return sp

    def _finish_reason(self, req) -> str:
        fr = self.engine.meta_info(req).get("finish_reason") or {}
        return {"length": "length", "abort": "abort"}.get(fr.get("type"), "stop")

    async def _chat_completions(self, request):
        """``POST /v1/chat/completions``: chat template -> generate -> one choice. ``continue_final_message`` resumes a
        partial assistant message (what callers send after an abort during a weight update)."""
        from aiohttp import web

        body = await self._json(request)
        messages = body.get("messages")
        if not messages or self.tokenizer is None:
            return web.json_response({"error": {"message": "messages and a server-side tokenizer are required"}}, status=400)
        cont = bool(body.get("continue_final_message")) and messages[-1].get("role") == "assistant"
        kw = {"tools": body["tools"]} if body.get("tools") else {}
        if cont:
            text = self.tokenizer.apply_chat_template(messages[:-1], tokenize=False, add_generation_prompt=True, **kw)
            text += messages[-1].get("content") or ""
        else:
            text = self.tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=True, **kw)
        ids = self.tokenizer.encode(text, add_special_tokens=False)
        req = await self._run_one(ids, self._openai_sampling(body), rid=body.get("rid"))
        content = self.tokenizer.decode(req.output_ids, skip_special_tokens=True)
        return web.json_response({
            "id": f"chatcmpl-{req.rid}", "object": "chat.completion", "created": int(time.time()),
            "model": body.get("model") or self.engine.args.model_path or "default",
            "choices": [{"index": 0, "message": {"role": "assistant", "content": content},
                         "finish_reason": self._finish_reason(req)}],
            "usage": {"prompt_tokens": len(ids), "completion_tokens": len(req.output_ids),
                      "total_tokens": len(ids) + len(req.output_ids)}})  # fmt: skip

    async def _completions(self, request):
        from aiohttp import web

        body = await self._json(request)
        prompt = body.get("prompt")
        if prompt is None or (isinstance(prompt, str) and self.tokenizer is None):
            return web.json_response({"error": {"message": "prompt (token ids, or text with a tokenizer) is required"}}, status=400)
        ids = self.tokenizer.encode(prompt, add_special_tokens=False) if isinstance(prompt, str) else list(prompt)
        req = await self._run_one(ids, self._openai_sampling(body), rid=body.get("rid"))
        text = self.tokenizer.decode(req.output_ids, skip_special_tokens=True) if self.tokenizer is not None else ""
        return web.json_response({
            "id": f"cmpl-{req.rid}", "object": "text_completion", "created": int(time.time()),
            "model": body.get("model") or self.engine.args.model_path or "default",
            "choices": [{"index": 0, "text": text, "token_ids": list(req.output_ids), "finish_reason": self._finish_reason(req)}],
            "usage": {"prompt_tokens": len(ids), "completion_tokens": len(req.output_ids),
                      "total_tokens": len(ids) + len(req.output_ids)}})  # fmt: skip

    async def _models(self, _request):
        from aiohttp import web

        name = self.engine.args.model_path or "default"
        return web.json_response({"object": "list", "data": [{"id": name, "object": "model", "owned_by": "slime_b200"}]})

    def _render(self, req) -> dict:
        text = ""
        if self.tokenizer is not None:
            text = self.tokenizer.decode(req.output_ids, skip_special_tokens=req.sampling.skip_special_tokens)
        meta = self.engine.meta_info(req)
        if not req.return_logprob:
            meta.pop("output_token_logprobs", None)
            meta.pop("input_token_logprobs", None)
        return {"text": text, "output_ids": list(req.output_ids), "meta_info": meta}

    async def _json(self, request) -> dict:
        try:
            return await request.json()
        except Exception:  # noqa: BLE001
            return {}

    def _ok(self, **kw):
        from aiohttp import web

        return web.json_response({"success": True, **kw})

    async def _health(self, request):
        from aiohttp import web

        return web.Response(text="ok")

    async def _health_generate(self, request):
        from aiohttp import web

        if "weights" in self.engine.released or "kv_cache" in self.engine.released:
            return web.Response(text="ok (offloaded)")
        ev = threading.Event()
        req = self.engine.add_request([0], SamplingParams(max_new_tokens=1, ignore_eos=True), done_event=ev)
        self._wake.set()
        ok = await asyncio.get_running_loop().run_in_executor(None, ev.wait, float(request.query.get("timeout", 20)))
        return web.Response(text="ok") if ok or req.finished() else web.Response(status=503, text="generation stuck")

    async def _abort(self, request):
        body = await self._json(request)
        n = self.engine.abort(body.get("rid"), bool(body.get("abort_all", False)))
        return self._ok(aborted=n)

    async def _loads(self, request):
        from aiohttp import web

        info = self.engine.loads()
        inflight = request.query.get("include") == "inflight"
        if inflight:
            now = time.time()
            info["inflight"] = {"running": [now - r.arrival for r in self.engine.running],
                                "waiting": [now - r.arrival for r in self.engine.waiting]}  # fmt: skip
        return web.json_response([{"dp_rank": 0, **info}])

    async def _flush(self, request):
        from aiohttp import web

        ok = self.engine.flush_cache()
        return web.Response(status=200 if ok else 400, text="Cache flushed." if ok else "Cache not flushed: requests in flight.")

    async def _pause(self, request):
        self.engine.pause_generation()
        return self._ok()

    async def _continue(self, request):
        self.engine.continue_generation()
        self._wake.set()
        return self._ok()

    async def _release(self, request):
        body = await self._json(request)
        self.engine.flush_cache()
        self.kv_store.clear()  # exported KV nobody has fetched yet goes with the cache it was copied from
        self.engine.release_memory_occupation(body.get("tags"))
        return self._ok()

    async def _resume(self, request):
        body = await self._json(request)
        self.engine.resume_memory_occupation(body.get("tags"))
        return self._ok()

    async def _update_from_tensor(self, request):
        """Payload: ``serialized_named_tensors`` = base64(torch.save([(name, tensor), ...])) per TP rank, or
        ``local_handle`` naming tensors registered in-process (colocated fast path)."""
        body = await self._json(request)
        blobs = body.get("serialized_named_tensors") or []
        named = []
        for blob in blobs[:1]:
            named += torch.load(io.BytesIO(base64.b64decode(blob)), weights_only=False)
        missing = self.engine.update_weights(named, body.get("weight_version"), bool(body.get("flush_cache", True)))
        if self.engine.device.type == "cuda":
            torch.cuda.synchronize()  # reply only after the copies retired: the producer may reuse its buffer
        return self._ok(missing=missing)

    async def _update_from_disk(self, request):
        body = await self._json(request)
        from slime_b200.checkpoint.hf_loader import SafetensorReader

        reader = SafetensorReader(body["model_path"])
        with self.engine.lock:
            idle_deadline = time.time() + 60
            while (self.engine.running or self.engine.prefilling) and time.time() < idle_deadline:
                await asyncio.sleep(0.01)
            missing = self.engine.update_weights(((n, reader.get(n)) for n in reader.keys() if not n.endswith("_scale_inv")),
                                                 body.get("weight_version"))  # fmt: skip
        return self._ok(message="weights reloaded", missing=missing)

    async def _pull_weights(self, request):
        body = await self._json(request)
        from slime_b200.weight_sync.local_checkpoint import pull_weights

        loop = asyncio.get_running_loop()
        base = body.get("base_dir") or getattr(self.engine.args, "model_path", None)  # version 0 = what the engine booted from
        version_dir = await loop.run_in_executor(None, pull_weights, body["local_checkpoint_dir"], body["source_dir"],
                                                 int(body["target_version"]), base)  # fmt: skip
        return self._ok(path=version_dir)

    async def _init_group(self, request):
        body = await self._json(request)
        from slime_b200.utils.distributed_utils import init_extra_process_group

        def make():
            return init_extra_process_group(
                backend=body.get("backend", "nccl"), init_method=f"tcp://{body['master_address']}:{body['master_port']}",
                world_size=body["world_size"], rank=body["rank_offset"], group_name=body["group_name"],
            )  # fmt: skip

        self._update_groups[body["group_name"]] = await asyncio.get_running_loop().run_in_executor(None, make)
        return self._ok()

    async def _destroy_group(self, request):
        body = await self._json(request)
        import torch.distributed as dist

        g = self._update_groups.pop(body.get("group_name"), None)
        if g is not None:
            dist.destroy_process_group(g)
        return self._ok()

    async def _update_from_distributed(self, request):
        body = await self._json(request)
        import torch.distributed as dist

        group = self._update_groups[body["group_name"]]

        def recv():
            named = []
            for n, dt, shape in zip(body["names"], body["dtypes"], body["shapes"]):
                t = torch.empty(shape, dtype=getattr(torch, dt), device=self.engine.device)
                dist.broadcast(t, 0, group=group)
                named.append((n, t))
            return self.engine.update_weights(named, body.get("weight_version"), bool(body.get("flush_cache", False)))

        missing = await asyncio.get_running_loop().run_in_executor(None, recv)
        return self._ok(missing=missing)

    async def _weight_version(self, request):
        from aiohttp import web

        return web.json_response({"weight_version": self.engine.get_weight_version()})

    async def _weights_checker(self, request):
        """snapshot -> reset_tensors -> compare: verifies that a sync rewrites every weight."""
        body = await self._json(request)
        action = body.get("action")
        w = self.engine.weights
        if action == "snapshot":
            self._weights_snapshot = [t.detach().clone() for t in w.tensors()]
        elif action == "reset_tensors":
            for t in w.tensors():
                t.normal_(0, 1) if t.is_floating_point() else t.zero_()
        elif action == "compare":
            assert self._weights_snapshot is not None, "no snapshot"
            bad = [i for i, (a, b) in enumerate(zip(self._weights_snapshot, w.tensors())) if not torch.equal(a, b)]
            if bad:
                from aiohttp import web

                return web.json_response({"success": False, "mismatched_tensors": bad}, status=400)
        else:
            return self._ok(success=False, message=f"unknown action {action}")
        return self._ok()

    async def _post_process_weights(self, request):
        """Quantised engines: restore -> load -> re-pack cycle around a sync; dense bf16 weights need nothing."""
        return self._ok()

    async def _profile(self, request):
        body = await self._json(request)
        if request.path.endswith("start_profile"):
            self._profiler = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA])
            self._profiler.__enter__()
            self._profile_dir = body.get("output_dir", "/tmp")
        elif getattr(self, "_profiler", None) is not None:
            self._profiler.__exit__(None, None, None)
            self._profiler.export_chrome_trace(f"{self._profile_dir}/engine_{self.port}_{int(time.time())}.json")
            self._profiler = None
        return self._ok()

    async def _server_info(self, request):
        from aiohttp import web

        a = self.engine.args
        info = {
            "model_path": a.model_path, "tp_size": a.tp_size, "dp_size": a.dp_size, "pp_size": a.pp_size, "ep_size": a.ep_size,
            "disaggregation_mode": a.disaggregation_mode, "weight_version": self.engine.get_weight_version(),
            "max_total_num_tokens": self.engine.num_pages * self.engine.page_size, "version": "slime_b200",
            "internal_states": [self.engine.loads()],
        }  # fmt: skip
        return web.json_response(info)

    async def _metrics(self, request):
        from aiohttp import web

        st, ld = self.engine.stats, self.engine.loads()
        lines = [
            f"sglang:num_running_reqs {ld['num_running_reqs']}", f"sglang:num_queue_reqs {ld['num_waiting_reqs']}",
            f"sglang:prompt_tokens_total {st['prefill_tokens']}", f"sglang:generation_tokens_total {st['decode_tokens']}",
            f"sglang:cached_tokens_total {st['cached_tokens']}", f"sglang:cache_hit_rate {ld['hit_rate']}",
            f"sglang:uptime_seconds {time.time() - self.started_at}",
        ]  # fmt: skip
        return web.Response(text="\n".join(lines) + "\n")

    # ------------------------------------------------------------------------------ lifecycle
    def build_app(self):
        from aiohttp import web

        app = web.Application(client_max_size=1 << 34)
        r = app.router
        r.add_post("/generate", self._generate)
        r.add_get("/disagg/kv/{rid}", self._kv_fetch)
        r.add_post("/v1/chat/completions", self._chat_completions)
        r.add_post("/v1/completions", self._completions)
        r.add_get("/v1/models", self._models)
        for path in ("/health", "/healthz"):
            r.add_get(path, self._health)
        r.add_get("/health_generate", self._health_generate)
        r.add_post("/abort_request", self._abort)
        for path in ("/v1/loads", "/get_load", "/get_loads"):
            r.add_get(path, self._loads)
        r.add_get("/flush_cache", self._flush)
        r.add_post("/flush_cache", self._flush)
        r.add_post("/pause_generation", self._pause)
        r.add_post("/continue_generation", self._continue)
        r.add_post("/release_memory_occupation", self._release)
        r.add_post("/resume_memory_occupation", self._resume)
        r.add_post("/update_weights_from_tensor", self._update_from_tensor)
        r.add_post("/update_weights_from_disk", self._update_from_disk)
        r.add_post("/pull_weights", self._pull_weights)
        r.add_post("/init_weights_update_group", self._init_group)
        r.add_post("/destroy_weights_update_group", self._destroy_group)
        r.add_post("/update_weights_from_distributed", self._update_from_distributed)
        for path in ("/get_weight_version", "/weight_version"):
            r.add_get(path, self._weight_version)
        r.add_post("/weights_checker", self._weights_checker)
        r.add_post("/post_process_weights", self._post_process_weights)
        r.add_post("/start_profile", self._profile)
        r.add_post("/stop_profile", self._profile)
        for path in ("/server_info", "/get_server_info", "/get_model_info"):
            r.add_get(path, self._server_info)
        r.add_get("/metrics", self._metrics)
        return app

    def start(self, block: bool = False):
        """Start the scheduler thread and the HTTP listener (its own event loop thread unless ``block``)."""
        from aiohttp import web

        self._thread = threading.Thread(target=self._scheduler_loop, daemon=True, name="engine-scheduler")
        self._thread.start()
        ready = threading.Event()

        def serve():
            self._loop = asyncio.new_event_loop()
            asyncio.set_event_loop(self._loop)
            self._runner = web.AppRunner(self.build_app(), access_log=None)
            self._loop.run_until_complete(self._runner.setup())
            site = web.TCPSite(self._runner, self.host, self.port)
            self._loop.run_until_complete(site.start())
            if not self.port and self._runner.addresses:  # port 0: the kernel chose
                self.port = int(self._runner.addresses[0][1])
            ready.set()
            self._loop.run_forever()

        if block:
            serve()
        else:
            self._http_thread = threading.Thread(target=serve, daemon=True, name="engine-http")
            self._http_thread.start()
            ready.wait(timeout=30)
        return self

    def shutdown(self):
        self._stop.set()
        self._wake.set()
        if self._loop is not None:
            async def _close():
                await self._runner.cleanup()

            fut = asyncio.run_coroutine_threadsafe(_close(), self._loop)
            try:
                fut.result(timeout=5)
            except Exception:  # noqa: BLE001
                pass
            self._loop.call_soon_threadsafe(self._loop.stop)

    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.port}"


def launch_server(server_args, model_config=None, tokenizer=None, weights_loader=None, block=True) -> EngineServer:
    """Process entry point: build the engine from ``ServerArgs`` and serve."""
    from slime_b200.models.config import ModelConfig

    cfg = model_config or ModelConfig.from_hf(server_args.model_path)
    device = torch.device("cuda", server_args.base_gpu_id) if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if tokenizer is None and server_args.model_path:
        try:
            from slime_b200.utils.processing_utils import load_tokenizer

            tokenizer = load_tokenizer(server_args.tokenizer_path or server_args.model_path)
        except Exception:  # noqa: BLE001
            tokenizer = None
    engine = Engine(cfg, server_args, device=device, tokenizer=tokenizer)
    if weights_loader is not None:
        weights_loader(engine)
    elif server_args.load_format == "dummy" or not server_args.model_path or server_args.model_path.startswith("preset:"):
        engine.weights.init_random(server_args.random_seed)
    else:
        from slime_b200.checkpoint.hf_loader import SafetensorReader

        reader = SafetensorReader(server_args.model_path)
        engine.update_weights(((n, reader.get(n)) for n in reader.keys() if not n.endswith("_scale_inv")))
    processor = None
    if cfg.vision is not None and server_args.model_path:
        from slime_b200.utils.processing_utils import load_processor

        processor = load_processor(server_args.tokenizer_path or server_args.model_path)
    return EngineServer(engine, server_args.host, server_args.port, tokenizer, processor).start(block=block)


if __name__ == "__main__":
    import argparse
    import dataclasses

    from slime_b200.engine.server_args import ServerArgs

    p = argparse.ArgumentParser("slime_b200.engine.http_server")
    for f in dataclasses.fields(ServerArgs):
        kind = {"int": int, "float": float, "bool": lambda s: s.lower() in ("1", "true", "yes")}.get(str(f.type).split(" ")[0], str)
        p.add_argument("--" + f.name.replace("_", "-"), type=kind, default=None)
    ns = {k: v for k, v in vars(p.parse_args()).items() if v is not None}
    launch_server(ServerArgs.from_kwargs(**ns), block=True)
