"""HTTP front of the continuous-batching server (standard library only).

The reference ends at a ``generate`` function per sequence (ferrotorch-llama/src/generation.rs:145-228, streamed
through a callback).  For serving, requests arrive concurrently and leave as they finish, so this module puts
:class:`~ferrotorch_b200.models.serving.ContinuousBatcher` behind three routes:

``POST /v1/completions``
    ``{"prompt": "text" | [token ids], "max_tokens": 16, "temperature": 0, "top_p": 1, "top_k": 0, "seed": null,
    "repetition_penalty": 1, "stop_token_ids": [], "lookahead": 0, "stream": false}`` (``lookahead``: look-up
    speculation of greedy requests).  The answer carries the generated ids, the
    text when a tokenizer is attached, the finish reason and token counts.  With ``"stream": true`` the answer is
    a ``text/event-stream``: one ``data: {...}`` event per token as the serving loop produces it, then
    ``data: [DONE]``.  A client that goes away in mid-stream cancels its request.
``GET /health``
    ``{"status": "ok", "running": n, "waiting": n}``.
``GET /metrics``
    Counters and gauges of the batcher in the Prometheus text format.

One thread runs the batcher's loop (the only thread that touches the model); every connection has a handler
thread that submits its request and waits on it.
"""
from __future__ import annotations

import json
import queue
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from .serving import ContinuousBatcher, Request, SamplingParams


class BadRequest(ValueError):
    pass


def parse_completion_request(body: dict, encode=None) -> tuple:
    """``(prompt ids, max_tokens, stop ids, SamplingParams, stream, lookahead)`` from the JSON body of a completion call."""
    if not isinstance(body, dict) or "prompt" not in body:
        raise BadRequest("the body must be a JSON object with a 'prompt'")
    prompt = body["prompt"]
    if isinstance(prompt, str):
        if encode is None:
            raise BadRequest("this server has no tokenizer: send the prompt as a list of token ids")
        prompt = encode(prompt)
    if not isinstance(prompt, list) or not prompt or not all(isinstance(t, int) and not isinstance(t, bool) and t >= 0 for t in prompt):
        raise BadRequest("'prompt' must be text or a non-empty list of token ids")
    try:
        sp = SamplingParams(float(body.get("temperature", 0.0)), int(body.get("top_k", 0)), float(body.get("top_p", 1.0)),
                            None if body.get("seed") is None else int(body["seed"]), float(body.get("repetition_penalty", 1.0)))
        sp.validate()
        max_tokens = int(body.get("max_tokens", 16))
        stops = tuple(int(t) for t in body.get("stop_token_ids", ()))
        lookahead = max(0, int(body.get("lookahead", 0)))
    except (TypeError, ValueError) as e:
        raise BadRequest(str(e)) from None
    if max_tokens < 1:
        raise BadRequest("'max_tokens' must be at least 1")
    return prompt, max_tokens, stops, sp, bool(body.get("stream", False)), lookahead


def prometheus_text(batcher: ContinuousBatcher) -> str:
    s, pool = batcher.stats, batcher.cache.pool
    rows = [("steps_total", "counter", s.steps), ("prefill_tokens_total", "counter", s.prefill_tokens),
            ("decode_tokens_total", "counter", s.decode_tokens), ("preemptions_total", "counter", s.preemptions),
            ("requests_finished_total", "counter", s.finished), ("prefix_hit_tokens_total", "counter", s.prefix_hit_tokens),
            ("speculated_tokens_total", "counter", s.spec_proposed), ("speculated_tokens_accepted_total", "counter", s.spec_accepted),
            ("requests_running", "gauge", len(batcher.running)), ("requests_waiting", "gauge", len(batcher.waiting)),
            ("kv_pages_used", "gauge", pool.num_used), ("kv_pages_total", "gauge", pool.num_total)]
    return "".join("# TYPE ferrotorch_serving_%s %s\nferrotorch_serving_%s %d\n" % (n, t, n, v) for n, t, v in rows)


class ServingApp:
    """``ServingApp(batcher, encode=..., decode=...).start()`` serves on ``host:port`` (port 0 picks a free one,
    read it from ``.port``); ``shutdown()`` drains the running requests and stops both threads."""

    def __init__(self, batcher: ContinuousBatcher, encode=None, decode=None, model_name: str = "ferrotorch-b200"):
        self.batcher, self.encode, self.decode, self.model_name = batcher, encode, decode, model_name
        self._stop = threading.Event()
        self._loop: threading.Thread | None = None
        self._http: ThreadingHTTPServer | None = None
        self._http_thread: threading.Thread | None = None
        self._next = 0
        self._lock = threading.Lock()
        self.loop_error: BaseException | None = None

    # ------------------------------------------------------------------ life cycle
    def _run_loop(self) -> None:
        try:
            self.batcher.serve_forever(self._stop)
        except BaseException as e:  # noqa: BLE001  (reported by /health and by every waiting handler)
            self.loop_error = e
            for r in list(self.batcher.running) + list(self.batcher.waiting):
                r.finish_reason = "error"
                r._done.set()

    def start(self, host: str = "127.0.0.1", port: int = 0) -> "ServingApp":
        app = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):                    # quiet: the metrics route is the log
                pass

            def do_GET(self):
                app._get(self)

            def do_POST(self):
                app._post(self)

        self._http = ThreadingHTTPServer((host, port), Handler)
        self._http.daemon_threads = True
        self.host, self.port = self._http.server_address[:2]
        self._loop = threading.Thread(target=self._run_loop, name="serving-loop", daemon=True)
        self._http_thread = threading.Thread(target=self._http.serve_forever, name="serving-http", daemon=True)
        self._loop.start()
        self._http_thread.start()
        return self

    def shutdown(self, timeout: float = 60.0) -> None:
        if self._http is not None:
            self._http.shutdown()
            self._http.server_close()
        self._stop.set()
        if self._loop is not None:
            self._loop.join(timeout)

    # ------------------------------------------------------------------ routes
    @staticmethod
    def _send(h, code: int, payload, content_type: str = "application/json") -> None:
        data = payload if isinstance(payload, bytes) else (payload if isinstance(payload, str) else json.dumps(payload)).encode()
        h.send_response(code)
        h.send_header("Content-Type", content_type)
        h.send_header("Content-Length", str(len(data)))
        h.end_headers()
        h.wfile.write(data)

    def _get(self, h) -> None:
        if h.path == "/health":
            ok = self.loop_error is None
            self._send(h, 200 if ok else 500, {"status": "ok" if ok else "error: %r" % (self.loop_error,),
                                              "running": len(self.batcher.running), "waiting": len(self.batcher.waiting)})
        elif h.path == "/metrics":
            self._send(h, 200, prometheus_text(self.batcher), "text/plain; version=0.0.4")
        else:
            self._send(h, 404, {"error": "no route %s" % h.path})

    def _choice(self, r: Request) -> dict:
        c = {"index": 0, "token_ids": list(r.output), "finish_reason": r.finish_reason}
        if self.decode is not None:
            c["text"] = self.decode(list(r.output))
        return c

    def _post(self, h) -> None:
        if h.path != "/v1/completions":
            return self._send(h, 404, {"error": "no route %s" % h.path})
        try:
            n = int(h.headers.get("Content-Length", "0"))
            body = json.loads(h.rfile.read(n) or b"null")
            prompt, max_tokens, stops, sp, stream, lookahead = parse_completion_request(body, self.encode)
            events: queue.Queue | None = queue.Queue() if stream else None
            req = Request(prompt, max_tokens, stops, sp, on_token=events.put if stream else None, lookahead=lookahead)
            self.batcher.submit(req)
        except (BadRequest, json.JSONDecodeError, ValueError, RuntimeError) as e:      # RuntimeError: the pool cannot hold it
            return self._send(h, 400, {"error": str(e)})
        with self._lock:
            rid, self._next = "cmpl-%d" % self._next, self._next + 1
        if not stream:
            while not req._done.wait(0.5):
                if self.loop_error is not None:           # the request was still in the inbox when the loop stopped
                    req.finish_reason = "error"
                    break
            if req.finish_reason == "error":
                return self._send(h, 500, {"error": "the serving loop stopped: %r" % (self.loop_error,)})
            return self._send(h, 200, {"id": rid, "object": "text_completion", "model": self.model_name, "choices": [self._choice(req)],
                                       "usage": {"prompt_tokens": len(req.prompt), "completion_tokens": len(req.output),
                                                 "total_tokens": len(req.prompt) + len(req.output)}})
        h.send_response(200)
        h.send_header("Content-Type", "text/event-stream")
        h.send_header("Cache-Control", "no-cache")
        h.send_header("Connection", "close")
        h.end_headers()
        sent = 0
        try:
            while True:
                try:
                    tok = events.get(timeout=0.05)
                except queue.Empty:
                    if (req._done.is_set() or self.loop_error is not None) and events.empty():
                        break
                    continue
                ev = {"id": rid, "index": sent, "token_id": tok}
                if self.decode is not None:
                    ev["text"] = self.decode([tok])
                h.wfile.write(b"data: " + json.dumps(ev).encode() + b"\n\n")
                h.wfile.flush()
                sent += 1
            h.wfile.write(b"data: " + json.dumps({"id": rid, "finish_reason": req.finish_reason, "completion_tokens": sent}).encode() + b"\n\n")
            h.wfile.write(b"data: [DONE]\n\n")
            h.wfile.flush()
        except (BrokenPipeError, ConnectionResetError):
            self.batcher.cancel(req)                      # nobody is listening any more
        h.close_connection = True


def main(argv=None) -> int:
    """``python -m ferrotorch_b200.models.server --model DIR [--device cuda] [--port 8000]``: serve a Hugging Face
    Llama directory (``config.json``, weights, ``tokenizer.json``).  ``--tiny`` serves a random tiny model on
    token ids (a smoke test that needs no files)."""
    import argparse
    import os
    import time

    import torch

    from .llama import LlamaConfig, LlamaForCausalLM

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--model")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--kv-pages", type=int, default=4096)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-running", type=int, default=64)
    ap.add_argument("--max-seq-len", type=int, default=None)
    ap.add_argument("--max-tokens-per-step", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--no-prefix-caching", action="store_true")
    ap.add_argument("--serve-seconds", type=float, default=None, help="stop after this long (default: until interrupted)")
    args = ap.parse_args(argv)
    if not args.tiny and not args.model:
        ap.error("give --model DIR or --tiny")
    dtype = torch.bfloat16 if args.device != "cpu" else torch.float32
    encode = decode = None
    if args.tiny:
        torch.manual_seed(0)
        model = LlamaForCausalLM(LlamaConfig.tiny()).to(device=args.device, dtype=dtype)
    else:
        model = LlamaForCausalLM.from_pretrained(args.model, dtype=dtype, device=args.device)
        tok_path = os.path.join(args.model, "tokenizer.json")
        if os.path.exists(tok_path):
            from ..utils import text

            tok = text.load_tokenizer(tok_path)
            encode, decode = (lambda s: text.encode(tok, s)), (lambda ids: text.decode(tok, ids))
    batcher = ContinuousBatcher(model.eval(), args.kv_pages, args.page_size, args.max_running,
                                args.max_seq_len or min(model.config.max_position_embeddings, args.kv_pages * args.page_size),
                                args.max_tokens_per_step, args.prefill_chunk, prefix_caching=not args.no_prefix_caching)
    app = ServingApp(batcher, encode, decode, os.path.basename(os.path.normpath(args.model)) if args.model else "tiny").start(args.host, args.port)
    print("serving on http://%s:%d (POST /v1/completions, GET /health, GET /metrics)" % (app.host, app.port), flush=True)
    try:
        t0 = time.monotonic()
        while app.loop_error is None and (args.serve_seconds is None or time.monotonic() - t0 < args.serve_seconds):
            time.sleep(0.05)
    except KeyboardInterrupt:
        pass
    finally:
        app.shutdown()
    return 0 if app.loop_error is None else 1


if __name__ == "__main__":
    raise SystemExit(main())
