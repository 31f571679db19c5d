"""OpenAI-compatible chat endpoint over a rollout engine, so agent frameworks that speak the chat
completions protocol can drive (and be trained through) the engine: ``POST /v1/chat/completions``,
``GET /v1/models``, ``GET /health`` (relax/components/rollout.py:907-973 proxy,
relax/agentic/session/service.py ``AgenticChatAPIService``).  Every completion is also appended to
the session named by the ``X-Session-Id`` header (or the ``user`` field), with token ids, loss mask and
log-probs, which is what turns API traffic into training samples.
"""
from __future__ import annotations

import json
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, Optional

from .agentic import GenerateFn, Session, SessionForest, Tokenizer


class ChatService:
    def __init__(self, generate: GenerateFn, tok: Tokenizer, model_name: str = "relax-b200-policy", max_context: int = 8192,
                 permits=None, abort_check=None):
        self.generate, self.tok, self.model_name, self.max_context = generate, tok, model_name, max_context
        # rollout.request_permit.InferencePermitManager: bounds the requests in flight across all front ends that
        # share the engines; a request that gets its permit after an abort was signalled raises GenerationAborted
        self.permits, self.abort_check = permits, abort_check
        self.forest = SessionForest()
        self.by_key: Dict[str, Session] = {}
        self._lock = threading.Lock()   # the engine is single-consumer

    def _session(self, key: Optional[str], messages: list) -> Session:
        prompt = []
        for m in messages:
            prompt += self.tok.encode(self.tok.render_turn(m["role"], m.get("content") or ""))
        prompt += self.tok.encode(self.tok.generation_prompt)
        s = self.by_key.get(key) if key else None
        if s is not None and prompt[:len(s.tokens)] == s.tokens:
            s.append(prompt[len(s.tokens):], 0)      # continuation of a known conversation: keep its generated tokens
            return s
        s = self.forest.new()
        s.append(prompt, 0)
        s.prompt_len = len(prompt)
        if key:
            self.by_key[key] = s
        return s

    def chat(self, body: dict, session_key: Optional[str] = None) -> dict:
        msgs = body.get("messages") or []
        if not msgs:
            raise ValueError("messages must be a non-empty list")
        n = int(body.get("n", 1))
        max_new = int(body.get("max_tokens") or body.get("max_completion_tokens") or 256)
        import contextlib

        gate = self.permits.permit(self.abort_check) if self.permits is not None else contextlib.nullcontext()
        with gate, self._lock:
            s = self._session(session_key or body.get("user"), msgs)
            room = self.max_context - len(s.tokens)
            if room <= 0:
                raise ValueError("conversation exceeds the context length")
            outs = self.generate([list(s.tokens)] * n, min(max_new, room), [s.sid] * n)
            toks, lps, reason, versions = outs[0]
            s.append(toks, 1, lps)
            s.weight_versions += versions
            s.turns += 1
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

    def finish_session(self, key: str, reward: float = 0.0):
        """Close a conversation and return it as a training sample."""
        s = self.by_key.pop(key)
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
