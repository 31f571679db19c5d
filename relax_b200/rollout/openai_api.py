"""OpenAI-compatible chat endpoint over a rollout engine, so agent frameworks that speak the chat
completions protocol can drive (and be trained through) the engine: ``POST /v1/chat/completions``,
``GET /v1/models``, ``GET /health`` (relax/components/rollout.py:907-973 proxy,
relax/agentic/session/service.py ``AgenticChatAPIService``).  Every completion is also appended to
the session named by the ``X-Session-Id`` header (or the ``user`` field), with token ids, loss mask and
log-probs, which is what turns API traffic into training samples.
"""
from __future__ import annotations

import contextlib
import json
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, Optional

from .agentic import GenerateFn, Session, SessionForest, Tokenizer


class ChatService:
    def __init__(self, generate: GenerateFn, tok: Tokenizer, model_name: str = "relax-b200-policy", max_context: int = 8192,
                 permits=None, abort_check=None, concurrent: bool = False, admission=None, on_gate=None):
        """``concurrent``: ``generate`` may be called from several threads at once (a batching backend joins the calls
        into one running batch), so only the session bookkeeping is serialised - needed when many agent processes talk
        to the endpoint.  ``admission`` (:class:`~relax_b200.rollout.admission.AdmissionController`): every completion
        first takes a token lease for its context plus the tokens it may generate
        (relax/agentic/session/admission.py).  ``on_gate(session_key, waiting)`` is told when a request starts and
        stops waiting for its lease (the owner pauses the agent's time budget meanwhile)."""
        self.generate, self.tok, self.model_name, self.max_context = generate, tok, model_name, max_context
        self.concurrent, self.admission, self.on_gate = concurrent, admission, on_gate
        self._busy: Dict[int, threading.Lock] = {}
        self._history: Dict[int, list] = {}       # session id -> [(role, content)] as exchanged with the client
        mark = "\x00"
        r = tok.render_turn("assistant", mark)
        self._turn_end = r[r.index(mark) + len(mark):] if mark in r else ""       # what closes an assistant turn
        # rollout.request_permit.InferencePermitManager: bounds the requests in flight across all front ends that
        # share the engines; a request that gets its permit after an abort was signalled raises GenerationAborted
        self.permits, self.abort_check = permits, abort_check
        self.forest = SessionForest()
        self.by_key: Dict[str, Session] = {}
        self._lock = threading.Lock()   # the engine is single-consumer

    def _session(self, key: Optional[str], messages: list) -> Session:
        """The session a request belongs to.  A request continues a known conversation when its message list starts
        with the messages already seen (compared as text, replies as they were returned): then the tokens kept for
        that part - the generated ones included, whose text need not re-tokenise to the same ids - stay, and only the
        new messages are rendered and appended."""
        turns = [(m["role"], m.get("content") or "") for m in messages]
        s = self.by_key.get(key) if key else None
        if s is not None:
            h = self._history.get(s.sid, [])
            if len(turns) > len(h) and turns[:len(h)] == h:
                text = self._turn_end if (h and h[-1][0] == "assistant") else ""
                text += "".join(self.tok.render_turn(r, c) for r, c in turns[len(h):]) + self.tok.generation_prompt
                s.append(self.tok.encode(text), 0)
                self._history[s.sid] = turns
                return s
        prompt = []
        for r, c in turns:
            prompt += self.tok.encode(self.tok.render_turn(r, c))
        prompt += self.tok.encode(self.tok.generation_prompt)
        s = self.forest.new()
        s.append(prompt, 0)
        s.prompt_len = len(prompt)
        self._history[s.sid] = turns
        if key:
            self.by_key[key] = s
        return s

    def chat(self, body: dict, session_key: Optional[str] = None) -> dict:
        msgs = body.get("messages") or []
        if not msgs:
            raise ValueError("messages must be a non-empty list")
        n = int(body.get("n", 1))
        max_new = int(body.get("max_tokens") or body.get("max_completion_tokens") or 256)
        gate = self.permits.permit(self.abort_check) if self.permits is not None else contextlib.nullcontext()
        key = session_key or body.get("user")
        if not self.concurrent:
            with gate, self._lock:
                s, outs = self._complete(key, msgs, n, max_new)
        else:
            with gate:
                s, outs = self._complete(key, msgs, n, max_new)
        toks = outs[0][0]
        choices = []
        for i, (t, lp, r, _) in enumerate(outs):
            c = {"index": i, "message": {"role": "assistant", "content": self.tok.decode(t)},
                 "finish_reason": "length" if r == "length" else "stop"}
            if body.get("logprobs"):
                c["logprobs"] = {"content": [{"token": self.tok.decode([a]), "logprob": b} for a, b in zip(t, lp)]}
            choices.append(c)
        ptoks = len(s.tokens) - len(toks)
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion", "created": int(time.time()),
                "model": body.get("model") or self.model_name, "choices": choices,
                "usage": {"prompt_tokens": ptoks, "completion_tokens": sum(len(o[0]) for o in outs),
                          "total_tokens": ptoks + sum(len(o[0]) for o in outs)}}

    def _complete(self, key, msgs, n: int, max_new: int):
        """Session lookup, lease, generation, bookkeeping.  In concurrent mode the service lock covers only the
        bookkeeping; two requests of the SAME session still run one after the other."""
        if self.concurrent:
            with self._lock:
                s = self._session(key, msgs)
                busy = self._busy.setdefault(s.sid, threading.Lock())
        else:
            s, busy = self._session(key, msgs), contextlib.nullcontext()
        with busy:
            room = self.max_context - len(s.tokens)
            if room <= 0:
                raise ValueError("conversation exceeds the context length")
            budget = min(max_new, room)
            lease = None
            if self.admission is not None:
                from .admission import reservation_tokens

                if self.on_gate is not None:
                    self.on_gate(key, True)
                try:
                    lease = self.admission.acquire(reservation_tokens(len(s.tokens), budget * n))
                finally:
                    if self.on_gate is not None:
                        self.on_gate(key, False)
            try:
                outs = self.generate([list(s.tokens)] * n, budget, [s.sid] * n)
            finally:
                if lease is not None:
                    self.admission.release(lease)
            toks, lps, reason, versions = outs[0]
            with (self._lock if self.concurrent else contextlib.nullcontext()):
                s.append(toks, 1, lps)
                s.weight_versions += versions
                s.turns += 1
                self._history.setdefault(s.sid, []).append(("assistant", self.tok.decode(toks)))
                if reason == "length" and budget == room:
                    s.truncated = True
        return s, outs

    def finish_session(self, key: str, reward: float = 0.0):
        """Close a conversation and return it as a training sample."""
        s = self.by_key.pop(key)
        self._history.pop(s.sid, None)
        self._busy.pop(s.sid, None)
        s.reward, s.done = reward, True
        return s.to_sample()


def serve(service: ChatService, host: str = "127.0.0.1", port: int = 0):
    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _reply(self, code, body):
            data = json.dumps(body).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def do_GET(self):
            if self.path == "/health":
                return self._reply(200, {"status": "ok"})
            if self.path == "/v1/models":
                return self._reply(200, {"object": "list", "data": [{"id": service.model_name, "object": "model"}]})
            self._reply(404, {"error": {"message": "unknown route", "type": "invalid_request_error"}})

        def do_POST(self):
            n = int(self.headers.get("Content-Length", "0"))
            try:
                body = json.loads(self.rfile.read(n) or b"{}")
                if self.path == "/v1/chat/completions":
                    if body.get("stream"):
                        raise ValueError("streaming responses are not supported")
                    return self._reply(200, service.chat(body, self.headers.get("X-Session-Id")))
                self._reply(404, {"error": {"message": "unknown route", "type": "invalid_request_error"}})
            except Exception as e:  # noqa: BLE001
                self._reply(400, {"error": {"message": f"{type(e).__name__}: {e}", "type": "invalid_request_error"}})

    srv = ThreadingHTTPServer((host, port), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv, f"http://{host}:{srv.server_address[1]}"
