"""The training model behind an HTTP endpoint: score token sequences (and optionally sample) with trainer numerics.

    python -m slime_b200.backends.train.server --hf-checkpoint /ckpt/teacher --load /ckpt/teacher --port 5000

Use: an on-policy-distillation teacher (``--rm-url http://host:5000/generate`` with
``slime.rollout.on_policy_distillation``), or a log-prob oracle whose arithmetic is exactly the trainer's.

    POST /generate   {"input_ids": [...], "sample_n": 0, "label_token_ids": [[...], ...]}
                     -> {"request_id", "log_probs": [T-1],                 log p(x_{t+1} | x_{<=t})
                         "label_token_log_probs": [T-1][K],                log p(label | x_{<=t}) for K given ids per position
                         "sampled_token_ids" / "sampled_log_probs": [T-1][sample_n],
                         "meta_info": {"input_token_logprobs": [[None, id0], [lp, id1], ...]}}   (engine-compatible view)
    POST /update_weights_from_disk {"model_path": ...}   waits until idle, reloads HF or torch_dist weights
    GET  /get_loads /info /healthz /detect

Requests are queued and packed: a worker thread drains the queue up to ``--max-tokens-per-gpu`` tokens, runs one
varlen forward (the model's own kernels, no grad), takes ``log_softmax`` of the fp32 logits and answers every request
of the pack. One process serves one data-parallel replica; put several behind the router for more throughput.
Parity: slime/backends/megatron_utils/server/megatron_server.py:82-603 and logprob_utils.py.
"""

from __future__ import annotations

import asyncio
import itertools
import logging
import threading
import time
from dataclasses import dataclass, field

import torch

logger = logging.getLogger(__name__)


@dataclass
class _Request:
    rid: str
    input_ids: list[int]
    sample_n: int = 0
    label_token_ids: list[list[int]] | None = None
    done: threading.Event = field(default_factory=threading.Event)
    result: dict | None = None
    error: str | None = None
    cancelled: bool = False


def parse_sample_n(v) -> int:
    if v is None or v is False:
        return 0
    n = int(v)
    if n < 0 or n > 64:
        raise ValueError("sample_n must be in [0, 64]")
    return n


def normalize_label_token_ids(labels, expected_length: int):
    """``[T-1][K]`` rectangular list of candidate ids per position, or None."""
    if labels is None:
        return None
    if not isinstance(labels, list) or len(labels) != expected_length:
        raise ValueError(f"label_token_ids must have one row per predicted position ({expected_length})")
    rows = [[int(x) for x in (r if isinstance(r, list) else [r])] for r in labels]
    if len({len(r) for r in rows}) > 1:
        raise ValueError("label_token_ids rows must all have the same length")
    return rows


class LogprobService:
    """Queue + packing worker around a model callable ``forward(ids[T], cu_seqlens) -> logits [T, V] fp32``."""

    def __init__(self, forward, max_tokens: int = 16384, temperature: float = 1.0, device="cpu", seed: int = 0):
        self.forward, self.max_tokens, self.temperature, self.device = forward, max_tokens, temperature, device
        self.queue: list[_Request] = []
        self.inflight = 0
        self.served = 0
        self.cv = threading.Condition()
        self.ids = itertools.count()
        self.running = True
        self.gen = torch.Generator(device=device).manual_seed(seed)
        self.thread = threading.Thread(target=self._loop, daemon=True, name="logprob-worker")
        self.thread.start()

    # ---------------------------------------------------------------- client side
    def submit(self, input_ids, sample_n=0, label_token_ids=None) -> _Request:
        r = _Request(f"req-{next(self.ids)}", list(input_ids), sample_n, label_token_ids)
        with self.cv:
            self.queue.append(r)
            self.cv.notify()
        return r

    def cancel(self, r: _Request):
        r.cancelled = True

    def loads(self) -> dict:
        with self.cv:
            return {"queue_size": len(self.queue), "inflight_size": self.inflight, "served": self.served,
                    "queued_tokens": sum(len(r.input_ids) for r in self.queue)}  # fmt: skip

    def wait_idle(self, timeout: float) -> bool:
        end = time.time() + timeout
        while time.time() < end:
            s = self.loads()
            if s["queue_size"] == 0 and s["inflight_size"] == 0:
                return True
            time.sleep(0.02)
        return False

    def stop(self):
        self.running = False
        with self.cv:
            self.cv.notify_all()
        self.thread.join(5)

    # ---------------------------------------------------------------- worker side
    def _take_pack(self) -> list[_Request]:
        with self.cv:
            while self.running and not self.queue:
                self.cv.wait(0.1)
            pack, used = [], 0
            while self.queue and (not pack or used + len(self.queue[0].input_ids) <= self.max_tokens):
                r = self.queue.pop(0)
                if r.cancelled:
                    continue
                pack.append(r)
                used += len(r.input_ids)
            self.inflight = len(pack)
            return pack

    def _loop(self):
        while self.running:
            pack = self._take_pack()
            if not pack:
                continue
            try:
                self._score(pack)
            except Exception as e:  # noqa: BLE001
                logger.exception("scoring a pack of %d requests failed", len(pack))
                for r in pack:
                    r.error = repr(e)
            for r in pack:
                r.done.set()
            with self.cv:
                self.inflight = 0
                self.served += len(pack)

    @torch.no_grad()
    def _score(self, pack: list[_Request]):
        lens = [len(r.input_ids) for r in pack]
        ids = torch.tensor([t for r in pack for t in r.input_ids], dtype=torch.long, device=self.device)
        cu = torch.tensor([0] + list(itertools.accumulate(lens)), dtype=torch.int32, device=self.device)
        logits = self.forward(ids, cu, max(lens)).float()
        if self.temperature != 1.0:
            logits = logits / self.temperature
        logp = torch.log_softmax(logits, dim=-1)
        off = 0
        for r, n in zip(pack, lens):
            lp = logp[off : off + n - 1] if n > 1 else logp[:0]  # row t predicts token t+1
            nxt = ids[off + 1 : off + n]
            out = {"log_probs": lp.gather(1, nxt[:, None]).squeeze(1).tolist() if n > 1 else []}
            if r.label_token_ids is not None and n > 1:
                lab = torch.tensor(r.label_token_ids, dtype=torch.long, device=self.device)
                out["label_token_log_probs"] = lp.gather(1, lab).tolist()
            if r.sample_n > 0 and n > 1:
                s = torch.multinomial(lp.exp(), r.sample_n, replacement=True, generator=self.gen)
                out["sampled_token_ids"] = s.tolist()
                out["sampled_log_probs"] = lp.gather(1, s).tolist()
            r.result = out
            off += n


def model_forward_fn(model):
    """Adapter: ``TrainModel`` (single pipeline stage) -> the callable ``LogprobService`` wants."""
    from slime_b200.models.gpt import PackedSeqParams

    chunk = model.chunks[0]
    chunk.eval()

    def forward(ids, cu, max_len):
        return chunk(ids, packed_seq_params=PackedSeqParams(cu, max_len))[0][:, : model.cfg.vocab_size]

    return forward


def build_app(service: LogprobService, info: dict, update_from_disk=None, max_request_length: int = 0):
    from aiohttp import web

    app = web.Application(client_max_size=64 * 1024 * 1024)
    state = {"updating": False}

    def err(msg, status):
        return web.json_response({"error": msg}, status=status)

    async def generate(request):
        if state["updating"]:
            return err("server is updating from disk", 503)
        try:
            body = await request.json()
        except Exception:  # noqa: BLE001
            return err("body is not JSON", 400)
        ids = body.get("input_ids")
        if not isinstance(ids, list) or not ids:
            return err("missing input_ids", 400)
        if max_request_length and len(ids) > max_request_length:
            return web.json_response({"error": f"input_ids length {len(ids)} exceeds configured maximum {max_request_length}",
                                      "input_length": len(ids), "max_length": max_request_length}, status=413)  # fmt: skip
        try:
            n = parse_sample_n(body.get("sample_n", 0))
            labels = normalize_label_token_ids(body.get("label_token_ids"), max(len(ids) - 1, 0))
        except ValueError as e:
            return err(str(e), 400)
        r = service.submit(ids, n, labels)
        try:
            while not r.done.is_set():
                await asyncio.sleep(0.002)
        except asyncio.CancelledError:  # client went away: do not spend a forward pass on it
            service.cancel(r)
            raise
        if r.error:
            return err(f"result failed: {r.error}", 500)
        out = {"request_id": r.rid, **r.result}
        out["meta_info"] = {"input_token_logprobs": [[None, ids[0]]] + [[lp, t] for lp, t in zip(out["log_probs"], ids[1:])],
                            "prompt_tokens": len(ids), "completion_tokens": 0}  # fmt: skip
        return web.json_response(out)

    async def update(request):
        body = await request.json()
        path = body.get("model_path") or body.get("path")
        if not path:
            return err("missing model_path", 400)
        if update_from_disk is None:
            return err("this server cannot reload weights", 501)
        if state["updating"]:
            return err("an update is already in progress", 409)
        state["updating"] = True
        try:
            timeout = float(body.get("timeout_s", 600))
            idle = await asyncio.get_running_loop().run_in_executor(None, service.wait_idle, timeout)
            if not idle:
                return err("server did not become idle in time", 504)
            await asyncio.get_running_loop().run_in_executor(None, update_from_disk, path)
            return web.json_response({"ok": True, "model_path": path})
        finally:
            state["updating"] = False

    def constant(make):
        async def handler(_request):
            return web.json_response(make())

        return handler

    app.router.add_get("/detect", constant(lambda: {"server_type": "slime_b200_train_server"}))
    app.router.add_get("/healthz", constant(lambda: {"ok": True}))
    app.router.add_get("/info", constant(lambda: {"args": info}))
    app.router.add_get("/get_loads", constant(service.loads))
    app.router.add_post("/update_weights_from_disk", update)
    app.router.add_post("/generate", generate)
    return app


def launch(args, block: bool = True):
    """Build the model from trainer args, load ``--load`` (or ``--hf-checkpoint``) and serve."""
    from aiohttp import web

    from slime_b200.backends.train import checkpoint as ckpt
    from slime_b200.backends.train.model import TrainModel
    from slime_b200.parallel import state as mpu

    if not mpu.model_parallel_is_initialized():
        mpu.initialize_model_parallel()
    model = TrainModel(args, with_optimizer=False)
    args.load = args.load or args.hf_checkpoint
    if args.load and not str(args.load).startswith("preset:"):
        ckpt.load_checkpoint(args, model, load_optimizer=False)

    def reload(path):
        from argparse import Namespace

        ckpt.load_checkpoint(Namespace(**{**vars(args), "load": path, "finetune": True}), model, load_optimizer=False)

    service = LogprobService(model_forward_fn(model), max_tokens=args.max_tokens_per_gpu or 16384,
                             temperature=getattr(args, "server_temperature", 1.0), device=model.device, seed=args.seed)  # fmt: skip
    info = {k: v for k, v in vars(args).items() if isinstance(v, (int, float, str, bool, type(None)))}
    app = build_app(service, info, reload, getattr(args, "server_max_request_length", 0) or 0)
    host, port = getattr(args, "server_host", "0.0.0.0"), getattr(args, "server_port", 5000)
    if block:
        web.run_app(app, host=host, port=port, access_log=None)
        return None
    return app, service


def main(argv=None):
    from slime_b200.utils.arguments import parse_args

    def extra(parser):
        g = parser.add_argument_group("train model server")
        g.add_argument("--server-host", default="0.0.0.0")
        g.add_argument("--server-port", type=int, default=5000)
        g.add_argument("--server-temperature", type=float, default=1.0)
        g.add_argument("--server-max-request-length", type=int, default=0)
        return parser

    launch(parse_args(argv, add_custom_arguments=extra))


if __name__ == "__main__":
    main()
