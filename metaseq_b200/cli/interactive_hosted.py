"""``metaseq-api-local``: HTTP completions service with dynamic batching.

Architecture (reference: metaseq/cli/interactive_hosted.py:66-431): every rank loads its model
part; rank 0 runs an HTTP server whose handler threads turn requests into ``WorkItem``s on a
keyed priority queue, and a batching thread that drains the fullest queue into batches
bounded by ``MAX_BATCH_TOKENS`` / ``MAX_SEQ_LEN``, broadcasts each batch's request object to
the other ranks and runs ``generator.generate``; the other ranks loop on that broadcast and
run the same generation so that tensor-parallel collectives line up.  A CUDA error in the
batching thread kills the process so that an external supervisor restarts it.

The HTTP layer uses the standard library (``http.server``) instead of Flask, which this
framework does not depend on; routes and JSON shapes are unchanged: ``POST /completions``
(also ``/v1/engines/<engine>/completions`` and ``/v2/...``), ``GET /`` for a tiny index page.
"""
from __future__ import annotations

import importlib
import json
import logging
import os
import queue
import random
import shutil
import threading
import time
import traceback
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import torch

from metaseq_b200 import options
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.hub_utils import GeneratorInterface
from metaseq_b200.parallel import utils as dist_utils
from metaseq_b200.service import constants as _default_constants
from metaseq_b200.service.queue import PriorityQueueRing
from metaseq_b200.service.responses import OAIResponse
from metaseq_b200.service.utils import build_logger, normalize_newlines
from metaseq_b200.service.workers import WorkItem


def _load_constants():
    name = os.environ.get("METASEQ_SERVICE_CONSTANTS_MODULE")
    if name:
        return importlib.import_module(name)
    return _default_constants


C = _load_constants()
logger = build_logger()
BATCH_QUEUE = PriorityQueueRing()
generator: GeneratorInterface = None
port = C.DEFAULT_PORT
_uid = [0]
_uid_lock = threading.Lock()


def next_uid() -> int:
    with _uid_lock:
        _uid[0] += 1
        return _uid[0]


def batching_loop(timeout=100, max_tokens=None, stop_event=None):
    """Collects queued work into batches and runs them.  A batch is dispatched when adding the next
    item would exceed ``max_tokens`` (longest prompt+generation times batch size) or when nothing
    new arrived for ``timeout`` ms."""
    max_tokens = max_tokens or C.MAX_BATCH_TOKENS
    batch_dict = None
    target_queue = None
    while stop_event is None or not stop_event.is_set():
        try:
            shard = BATCH_QUEUE.largest_shard()
            timeout_s = timeout / 1000 if batch_dict else 0.2
            if target_queue is None:
                target_queue = shard.get_deepest_queue()
            if target_queue is None:
                time.sleep(min(timeout_s, 0.05))
                raise queue.Empty
            item = target_queue.get(timeout=timeout_s)
            shard.size -= 1
            if batch_dict is None:
                batch_dict = {"items": [], "max_prompt_len": 0, "max_gen_len": 0}
            new_prompt = max(batch_dict["max_prompt_len"], item.prompt_len)
            new_gen = max(batch_dict["max_gen_len"], item.gen_len)
            overflow = (len(batch_dict["items"]) + 1) * (new_prompt + new_gen) > max_tokens or \
                new_prompt + new_gen > C.MAX_SEQ_LEN
            if overflow and batch_dict["items"]:
                target_queue.put(item)
                shard.size += 1
                raise queue.Empty
            batch_dict["items"].append(item)
            batch_dict["max_prompt_len"], batch_dict["max_gen_len"] = new_prompt, new_gen
        except queue.Empty:
            target_queue = None
            if batch_dict and batch_dict["items"]:
                _run_batch(batch_dict["items"])
                batch_dict = None


def _run_batch(items):
    request_object = {"inputs": [], "min_tokens": [], "max_tokens": []}
    for work in items:
        ro = work.data
        request_object["inputs"].append(ro["input"])
        request_object["min_tokens"].append(ro.get("min_tokens", 0))
        request_object["max_tokens"].append(ro.get("max_tokens", C.MAX_SEQ_LEN))
        for key in ro:
            if key not in ("input", "min_tokens", "max_tokens"):
                request_object[key] = ro[key]
    if "seed" not in request_object:
        request_object["seed"] = random.randint(1, 20000)
    if torch.distributed.is_initialized():
        dist_utils.broadcast_object(request_object, src_rank=0, group=dist_utils.get_global_group())
    try:
        generations = generator.generate(**request_object)
    except RuntimeError:
        # a device-side failure leaves the ranks out of step: exit hard so the supervisor restarts us
        logger.error("generation failed; terminating the worker:\n" + traceback.format_exc())
        os._exit(1)
    except BaseException as e:
        generations = [e] * len(items)
    for work, gen in zip(items, generations):
        work.return_queue.put((work.uid, gen))


def worker_main(cfg1, namespace_args=None):
    """Per-rank entry: load the model, then serve (rank 0) or follow broadcasts (other ranks)."""
    global generator, port
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    generator = GeneratorInterface(cfg1)
    models = generator.load_model()
    logger.info(f"loaded model {cfg1.distributed_training.distributed_rank}")
    if not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0:
        logger.info(f"Worker engaged! {get_my_ip()}:{port}")
        thread = threading.Thread(target=batching_loop, daemon=True)
        thread.start()
        server = ThreadingHTTPServer(("0.0.0.0", port), CompletionsHandler)
        server.serve_forever()
    else:
        logger.info(f"Looping engaged! {get_my_ip()}:{port}")
        while True:
            try:
                request_object = dist_utils.broadcast_object(None, src_rank=0, group=dist_utils.get_global_group())
                _ = generator.generate(**request_object)
            except Exception:
                logger.error("follower rank failed:\n" + traceback.format_exc())
                os._exit(1)


def get_my_ip():
    import socket

    try:
        return socket.gethostbyname(socket.gethostname())
    except OSError:
        return "127.0.0.1"


def _create_error_response(msg, http_code, **others):
    return {"error": {"message": msg, "type": "invalid_request_error" if http_code < 500 else "oops", **others}}, http_code


def validate_key(authorization: str) -> bool:
    """Any non-placeholder bearer token is accepted; deployments plug real checks in here."""
    return authorization not in ("Bearer YOUR_API_KEY", "Bearer ")


def handle_completions(body: dict, headers: dict):
    """Pure function behind ``POST /completions``: normalises the request, enqueues one work item
    per prompt and waits for the results.  Returns ``(json_dict, http_status)``."""
    auth = headers.get("Authorization") or headers.get("authorization")
    if auth is not None and not validate_key(auth):
        return _create_error_response("Invalid API key or API key missing.", 401)
    prompts = body.get("prompt")
    del_prompt_keys = True
    if prompts is None:
        return _create_error_response("prompt is required", 400)
    if isinstance(prompts, str):
        prompts = [prompts]  # single string
    elif isinstance(prompts, list) and len(prompts) > 0 and isinstance(prompts[0], int):
        prompts = [prompts]  # single pre-tokenised prompt
    assert isinstance(prompts, list)
    if len(prompts) == 0:
        return _create_error_response("prompt must not be empty", 400)
    if isinstance(prompts[0], str):
        prompts = [generator.encode_fn(normalize_newlines(p)) for p in prompts]
    go = {k: v for k, v in body.items() if k != "prompt"}
    if "min_tokens" in go:
        go["min_tokens"] = int(go["min_tokens"])
    if "max_tokens" in go:
        go["max_tokens"] = int(go["max_tokens"])
    if "stop" in go:
        stop = go["stop"]
        if stop is None:
            del go["stop"]
        else:
            if isinstance(stop, str):
                stop = [stop]
            go["stop"] = [generator.encode_fn(s)[0] for s in stop]
    if "temperature" in go:
        go["temperature"] = round(float(go["temperature"]), 1)
    else:
        go["temperature"] = 1.0
    if "top_p" in go:
        go["top_p"] = round(float(go["top_p"]), 1)
    else:
        go["top_p"] = 1.0
    go["n"] = min(int(go.get("n", 1)), C.MAX_BEAM)
    go["best_of"] = min(int(go.get("best_of", go["n"])), C.MAX_BEAM)
    go["best_of"] = max(go["best_of"], go["n"])
    if "logprobs" in go:
        go["logprobs"] = int(go["logprobs"])
    else:
        go["logprobs"] = 0
    for k in ("omega_bound", "lambda_decay", "alpha_presence", "alpha_frequency", "alpha_presence_src",
              "alpha_frequency_src"):
        if k in go:
            go[k] = float(go[k])
    if "alpha_src_penalty_end_idx" in go:
        go["alpha_src_penalty_end_idx"] = int(go["alpha_src_penalty_end_idx"])
    go.pop("model", None)
    go.pop("stream", None)
    go.pop("user", None)
    ret_queue: "queue.Queue" = queue.Queue()
    for i, prompt in enumerate(prompts):
        gen_len = go.get("max_tokens", 0)
        if gen_len + len(prompt) + 1 > C.MAX_SEQ_LEN:
            # keep the end of the prompt so that prompt + generation fits the position table
            cut = C.MAX_SEQ_LEN - gen_len - 1
            if cut <= 0:
                return _create_error_response("max_tokens is too large for the model's context", 400)
            prompt = prompt[-cut:]
        request_object = {"input": prompt, **go}
        BATCH_QUEUE.put(WorkItem(cost=len(prompt) + gen_len, uid=i, return_queue=ret_queue, data=request_object,
                                 prompt_len=len(prompt), gen_len=gen_len))
    unordered = []
    for _ in prompts:
        unordered.append(ret_queue.get())
    reordered = sorted(unordered, key=lambda x: x[0])
    results = []
    for uid, generations in reordered:
        if isinstance(generations, Exception):
            return _create_error_response(str(generations), 500)
        results += generations
    return OAIResponse(results).to_dict(), 200


_INDEX = """<html><body><h2>metaseq_b200 completions service</h2>
<form onsubmit="event.preventDefault();fetch('/completions',{method:'POST',headers:{'Content-Type':'application/json'},
body:JSON.stringify({prompt:document.getElementById('p').value,max_tokens:32,temperature:0.7,top_p:0.9})})
.then(r=>r.json()).then(j=>{document.getElementById('o').textContent=JSON.stringify(j,null,1)})">
<textarea id=p rows=4 cols=80></textarea><br><input type=submit value=Complete></form><pre id=o></pre></body></html>"""


class CompletionsHandler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"

    def log_message(self, fmt, *args):
        logger.info("%s - %s" % (self.address_string(), fmt % args))

    def _send(self, code, payload, content_type="application/json"):
        data = payload if isinstance(payload, bytes) else (
            payload.encode("utf-8") if isinstance(payload, str) else json.dumps(payload).encode("utf-8"))
        self.send_response(code)
        self.send_header("Content-Type", content_type)
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)

    def do_GET(self):
        if self.path in ("/", "/index.html"):
            return self._send(200, _INDEX, "text/html")
        return self._send(404, {"error": {"message": "not found"}})

    def do_POST(self):
        path = self.path.split("?")[0].rstrip("/")
        ok = path.endswith("/completions") and (path == "/completions" or path.startswith("/v1/engines/")
                                                or path.startswith("/v2/engines/"))
        if not ok:
            return self._send(404, {"error": {"message": "not found"}})
        try:
            n = int(self.headers.get("Content-Length", "0"))
            body = json.loads(self.rfile.read(n) or b"{}")
        except (ValueError, json.JSONDecodeError):
            return self._send(400, {"error": {"message": "request body must be JSON"}})
        try:
            payload, code = handle_completions(body, dict(self.headers))
        except Exception as e:
            logger.error(traceback.format_exc())
            payload, code = _create_error_response(str(e), 500, stacktrace=traceback.format_tb(e.__traceback__))
        return self._send(code, payload)


def cli_main():
    """Command-line entry point: ``LAUNCH_ARGS`` from the constants module form the argv."""
    global port
    parser = options.get_generation_parser()
    flat_launch_args = []
    for s in C.LAUNCH_ARGS:
        flat_launch_args += s.split()
    args = options.parse_args_and_arch(parser, input_args=flat_launch_args)
    args.data = os.path.dirname(args.path)  # hardcode the data arg
    port = C.DEFAULT_PORT
    cfg = convert_namespace_to_config(args)
    cfg.distributed_training.distributed_world_size = C.TOTAL_WORLD_SIZE
    dist_utils.call_main(cfg, worker_main, namespace_args=args)


if __name__ == "__main__":
    cli_main()
