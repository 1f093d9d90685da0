"""OpenAI-compatible chat front for a checkpoint under evaluation: strict request validation and a
ticket queue that the generation loop drains at a collective boundary, so HTTP threads never touch
the model (src/archlab/serving/openai_chat.py:23-300).

``"stream": true`` is answered as server-sent events (``chat.completion.chunk`` objects, then ``data: [DONE]``): the
generation loop calls ``Ticket.emit(piece)`` as text becomes available and the HTTP thread forwards every piece at once
with buffering switched off for proxies, which is what a streaming playground needs from the server side (the
reference patches the MLflow UI to consume such a stream, src/archlab/serving/mlflow_playground_overlay.py:1-156; the
UI patch itself has no counterpart here, MLflow is not part of this framework)."""
from __future__ import annotations

import json
import math
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer


def validate_request(value, models: dict[str, str], *, max_tokens: int = 256) -> dict:
    if not isinstance(value, dict) or value.get("model") not in models:
        raise ValueError("choose a served checkpoint model")
    messages = value.get("messages")
    if not isinstance(messages, list) or not messages or len(messages) > 64:
        raise ValueError("messages must contain 1-64 text messages")
    clean = []
    for m in messages:
        role, content = m.get("role"), m.get("content")
        if role not in ("system", "user", "assistant"):
            raise ValueError("this endpoint supports text chat without tools")
        if isinstance(content, list):
            if not all(isinstance(x, dict) and x.get("type") == "text" and isinstance(x.get("text"), str) for x in content):
                raise ValueError("only text content is supported")
            content = "".join(x["text"] for x in content)
        if not isinstance(content, str):
            raise ValueError("message content must be text")
        clean.append({"role": role, "content": content})
    if clean[-1]["role"] != "user":
        raise ValueError("the final message must be from the user")
    limit = value.get("max_completion_tokens", value.get("max_tokens", 128))
    if type(limit) is not int or not 1 <= limit <= max_tokens:
        raise ValueError(f"max_tokens must be between 1 and {max_tokens}")
    temperature, top_p = value.get("temperature", 0.0), value.get("top_p", 1.0)
    if not isinstance(temperature, (int, float)) or not math.isfinite(temperature) or not 0 <= temperature <= 2:
        raise ValueError("temperature must be finite and in 0..2")
    if not isinstance(top_p, (int, float)) or not math.isfinite(top_p) or not 0 < top_p <= 1:
        raise ValueError("top_p must be in (0,1]")
    if value.get("n", 1) != 1 or value.get("tools") or value.get("stop"):
        raise ValueError("only one text completion without tools or custom stops is supported")
    seed = value.get("seed", 42)
    if type(seed) is not int or not -(2 ** 63) <= seed < 2 ** 64:
        raise ValueError("seed must fit the generator range")
    return {"model": value["model"], "variant": models[value["model"]], "messages": clean, "max_tokens": limit,
            "temperature": float(temperature), "top_p": float(top_p), "seed": seed, "stream": bool(value.get("stream", False))}


@dataclass
class Ticket:
    request: dict
    id: str = field(default_factory=lambda: "chatcmpl-" + uuid.uuid4().hex[:24])
    done: threading.Event = field(default_factory=threading.Event)
    text: str | None = None
    error: str | None = None
    pieces: "queue.Queue[str | None]" = field(default_factory=queue.Queue)      # streamed text; None closes the stream

    def emit(self, piece: str) -> None:
        """Streaming: hand the next piece of generated text to the waiting HTTP thread."""
        if piece:
            self.pieces.put(piece)

    def finish(self, text: str | None = None, error: str | None = None) -> None:
        self.text, self.error = text, error
        self.pieces.put(None)
        self.done.set()


class ChatFront:
    """``tickets`` is drained by the owner of the model: ``t = front.next_ticket(); t.finish(generate(t.request))``."""

    def __init__(self, host: str, port: int, token: str, models: dict[str, str], *, max_tokens: int = 256, timeout: float = 600.0):
        self.models, self.max_tokens, self.timeout, self.token = models, max_tokens, timeout, token
        self.tickets: queue.Queue[Ticket] = queue.Queue()
        self.state = {"phase": "starting"}
        front = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a):            # quiet
                pass

            def _send(self, code, payload):
                body = json.dumps(payload).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def _event(self, payload) -> None:
                self.wfile.write(b"data: " + (payload if isinstance(payload, bytes) else json.dumps(payload).encode()) + b"\n\n")
                self.wfile.flush()

            def _stream(self, t, req):
                """Server-sent events: a role chunk, one chunk per emitted piece, a finish chunk, ``[DONE]``."""
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("X-Accel-Buffering", "no")            # reverse proxies must not hold chunks back
                self.send_header("Connection", "close")
                self.end_headers()
                chunk = lambda delta, finish=None: {"id": t.id, "object": "chat.completion.chunk", "created": int(time.time()),
                                                    "model": req["model"], "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
                self._event(chunk({"role": "assistant"}))
                sent, deadline = "", time.monotonic() + front.timeout
                try:
                    while True:
                        try:
                            piece = t.pieces.get(timeout=max(0.0, deadline - time.monotonic()))
                        except queue.Empty:
                            self._event({"error": {"message": "generation timed out"}})
                            break
                        if piece is None:
                            if t.error:
                                self._event({"error": {"message": t.error}})
                            else:
                                rest = (t.text or "")[len(sent):] if (t.text or "").startswith(sent) else ""
                                if rest:                                  # a loop that never called emit still streams once
                                    self._event(chunk({"content": rest}))
                                self._event(chunk({}, "stop"))
                            break
                        sent += piece
                        self._event(chunk({"content": piece}))
                    self._event(b"[DONE]")
                except (BrokenPipeError, ConnectionResetError):
                    pass                                                  # the client went away; the ticket finishes on its own

            def do_GET(self):
                if self.path == "/v1/models":
                    self._send(200, {"object": "list", "data": [{"id": m, "object": "model"} for m in front.models]})
                elif self.path == "/health":
                    self._send(200, front.snapshot())
                else:
                    self._send(404, {"error": {"message": "not found"}})

            def do_POST(self):
                if self.headers.get("Authorization") != f"Bearer {front.token}":
                    return self._send(401, {"error": {"message": "invalid token"}})
                if self.path != "/v1/chat/completions":
                    return self._send(404, {"error": {"message": "not found"}})
                try:
                    n = int(self.headers.get("Content-Length", "0"))
                    req = validate_request(json.loads(self.rfile.read(n)), front.models, max_tokens=front.max_tokens)
                except (ValueError, json.JSONDecodeError) as e:
                    return self._send(400, {"error": {"message": str(e)}})
                t = Ticket(req)
                front.tickets.put(t)
                if req["stream"]:
                    return self._stream(t, req)
                if not t.done.wait(front.timeout):
                    return self._send(504, {"error": {"message": "generation timed out"}})
                if t.error:
                    return self._send(500, {"error": {"message": t.error}})
                self._send(200, {"id": t.id, "object": "chat.completion", "created": int(time.time()), "model": req["model"],
                                 "choices": [{"index": 0, "finish_reason": "stop",
                                              "message": {"role": "assistant", "content": t.text}}]})

        self.server = ThreadingHTTPServer((host, port), Handler)
        self.thread = threading.Thread(target=self.server.serve_forever, daemon=True)
        self.thread.start()
        self.state = {"phase": "serving"}

    @property
    def port(self) -> int:
        return self.server.server_address[1]

    def next_ticket(self, timeout: float | None = None) -> Ticket | None:
        try:
            return self.tickets.get(timeout=timeout)
        except queue.Empty:
            return None

    def set_state(self, phase: str, **meta) -> None:
        self.state = {"phase": phase, **meta}

    def snapshot(self) -> dict:
        return {**self.state, "queued": self.tickets.qsize()}

    def close(self) -> None:
        self.server.shutdown()
        self.server.server_close()
