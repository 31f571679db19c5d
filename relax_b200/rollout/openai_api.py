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
import re
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, Optional

from .agentic import GenerateFn, Session, SessionForest, Tokenizer


# --------------------------------------------------------------------------- parsers of the model's text
_TOOL_TAG = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def parse_tool_calls(text: str, parser: str):
    """``(content, tool_calls)``: calls the model wrote in the format of ``parser`` are cut out of the text.
    ``hermes`` / ``qwen`` / ``qwen25``: ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` blocks;
    ``json``: the whole reply is one ``{"name": ..., "arguments"|"parameters": ...}`` object (Llama-3 style).
    A block that is not valid JSON stays in the content (the agent sees what the model wrote)."""
    calls = []
    if parser in ("hermes", "qwen", "qwen25", "qwen3"):
        def take(m):
            try:
                obj = json.loads(m.group(1))
                if not isinstance(obj, dict) or "name" not in obj:
                    return m.group(0)
            except ValueError:
                return m.group(0)
            calls.append(obj)
            return ""

        text = _TOOL_TAG.sub(take, text)
    elif parser in ("json", "llama3"):
        try:
            obj = json.loads(text.strip())
            if isinstance(obj, dict) and "name" in obj:
                calls.append(obj)
                text = ""
        except ValueError:
            pass
    else:
        raise ValueError(f"unknown tool-call parser {parser!r} (hermes, qwen, qwen25, qwen3, json, llama3)")
    out = []
    for c in calls:
        args = c.get("arguments", c.get("parameters", {}))
        out.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                    "function": {"name": str(c["name"]), "arguments": args if isinstance(args, str) else json.dumps(args)}})
    return text.strip() if out else text, out


def split_reasoning(text: str, parser: str):
    """``(reasoning, rest)`` for models that think inside ``<think> ... </think>`` (``qwen3``, ``deepseek-r1``); an
    unterminated block (the reply was cut off while thinking) is all reasoning."""
    if parser not in ("qwen3", "deepseek-r1", "deepseek_r1", "think"):
        raise ValueError(f"unknown reasoning parser {parser!r} (qwen3, deepseek-r1)")
    t = text.lstrip()
    if t.startswith("<think>"):
        t = t[len("<think>"):]
    elif "</think>" not in t:
        return None, text
    if "</think>" in t:
        a, b = t.split("</think>", 1)
        return a.strip(), b.lstrip("\n")
    return t.strip(), ""


def _calls_sig(tool_calls) -> str:
    """What identifies the tool calls of a message when a client sends it back."""
    if not tool_calls:
        return ""
    out = []
    for c in tool_calls:
        f = c.get("function", c)
        a = f.get("arguments", "")
        out.append((f.get("name"), a if isinstance(a, str) else json.dumps(a)))
    return json.dumps(out)


class ChatService:
    def __init__(self, generate: GenerateFn, tok: Tokenizer, model_name: str = "relax-b200-policy", max_context: int = 8192,
                 permits=None, abort_check=None, concurrent: bool = False, admission=None, on_gate=None,
                 tool_call_parser: Optional[str] = None, reasoning_parser: Optional[str] = None):
        """``concurrent``: ``generate`` may be called from several threads at once (a batching backend joins the calls
        into one running batch), so only the session bookkeeping is serialised - needed when many agent processes talk
        to the endpoint.  ``admission`` (:class:`~relax_b200.rollout.admission.AdmissionController`): every completion
        first takes a token lease for its context plus the tokens it may generate
        (relax/agentic/session/admission.py).  ``on_gate(session_key, waiting)`` is told when a request starts and
        stops waiting for its lease (the owner pauses the agent's time budget meanwhile)."""
        self.generate, self.tok, self.model_name, self.max_context = generate, tok, model_name, max_context
        self.concurrent, self.admission, self.on_gate = concurrent, admission, on_gate
        # --agentic-tool-call-parser / --agentic-reasoning-parser: how replies are split into content, tool calls and
        # reasoning for the client (the recorded tokens are always the model's full text)
        self.tool_call_parser, self.reasoning_parser = tool_call_parser, reasoning_parser
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

    def _session(self, key: Optional[str], messages: list, tools=None) -> Session:
        """The session a request belongs to.  A request continues a known conversation when its message list starts
        with the messages already seen (compared as text, replies as they were returned): then the tokens kept for
        that part - the generated ones included, whose text need not re-tokenise to the same ids - stay, and only the
        new messages are rendered and appended."""
        turns = [(m["role"], m.get("content") or "", _calls_sig(m.get("tool_calls"))) for m in messages]

        def render(t):
            role, content, calls = t
            if calls:         # an assistant turn with tool calls that did not come from this session's own tokens
                content += "".join(f'\n<tool_call>{json.dumps({"name": n, "arguments": a})}</tool_call>' for n, a in json.loads(calls))
            return self.tok.render_turn(role, content)

        s = self.by_key.get(key) if key else None
        if s is not None:
            h = self._history.get(s.sid, [])
            if len(turns) > len(h) and turns[:len(h)] == h:
                text = self._turn_end if (h and h[-1][0] == "assistant") else ""
                text += "".join(render(t) for t in turns[len(h):]) + self.tok.generation_prompt
                s.append(self.tok.encode(text), 0)
                self._history[s.sid] = turns
                return s
        prompt = []
        if tools:
            prompt += self.tok.encode(self.tok.render_turn("tools", json.dumps(tools, sort_keys=True)))
        for t in turns:
            prompt += self.tok.encode(render(t))
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
        tools = body.get("tools") or None
        if not self.concurrent:
            with gate, self._lock:
                s, outs, first = self._complete(key, msgs, n, max_new, tools)
        else:
            with gate:
                s, outs, first = self._complete(key, msgs, n, max_new, tools)
        toks = outs[0][0]
        choices = []
        for i, (t, lp, r, _) in enumerate(outs):
            msg = first if i == 0 else self._message(self.tok.decode(t), bool(tools))
            c = {"index": i, "message": msg,
                 "finish_reason": "length" if r == "length" else ("tool_calls" if msg.get("tool_calls") else "stop")}
            if body.get("logprobs"):
                c["logprobs"] = {"content": [{"token": self.tok.decode([a]), "logprob": b} for a, b in zip(t, lp)]}
            choices.append(c)
        ptoks = len(s.tokens) - len(toks)
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion", "created": int(time.time()),
                "model": body.get("model") or self.model_name, "choices": choices,
                "usage": {"prompt_tokens": ptoks, "completion_tokens": sum(len(o[0]) for o in outs),
                          "total_tokens": ptoks + sum(len(o[0]) for o in outs)}}

    def _message(self, text: str, has_tools: bool) -> dict:
        """The assistant message a client receives for the model's ``text``."""
        msg = {"role": "assistant", "content": text}
        if self.reasoning_parser:
            thought, rest = split_reasoning(text, self.reasoning_parser)
            if thought is not None:
                msg["reasoning_content"], msg["content"] = thought, rest
        if self.tool_call_parser and has_tools:
            content, calls = parse_tool_calls(msg["content"], self.tool_call_parser)
            if calls:
                msg["content"], msg["tool_calls"] = (content or None), calls
        return msg

    def _complete(self, key, msgs, n: int, max_new: int, tools=None):
        """Session lookup, lease, generation, bookkeeping.  In concurrent mode the service lock covers only the
        bookkeeping; two requests of the SAME session still run one after the other."""
        if self.concurrent:
            with self._lock:
                s = self._session(key, msgs, tools)
                busy = self._busy.setdefault(s.sid, threading.Lock())
        else:
            s, busy = self._session(key, msgs, tools), contextlib.nullcontext()
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
                first = self._message(self.tok.decode(toks), bool(tools))
                # the client sends back what it received: that, not the raw text, identifies the turn
                self._history.setdefault(s.sid, []).append(("assistant", first.get("content") or "", _calls_sig(first.get("tool_calls"))))
                if reason == "length" and budget == room:
                    s.truncated = True
        return s, outs, first

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
            path = self.path.split("?")[0].rstrip("/") or "/"
            if path in ("/health", "/healthz"):
                return self._reply(200, {"status": "ok", "ok": True})
            if path in ("/v1/models", "/models"):
                return self._reply(200, {"object": "list", "data": [{"id": service.model_name, "object": "model", "created": 0,
                                                                    "owned_by": "relax_b200"}]})
            if path == "/debug_state":      # relax/agentic/session/service.py:2251: what the service holds right now
                ss = list(service.forest.sessions.values())
                return self._reply(200, {"session_count": len(ss), "open_sessions": len(service.by_key),
                                         "turns": sum(s_.turns for s_ in ss), "tokens": sum(len(s_.tokens) for s_ in ss),
                                         "admission": service.admission.metrics() if service.admission is not None else None})
            self._reply(404, {"error": {"message": "unknown route", "type": "invalid_request_error"}})

        def do_POST(self):
            n = int(self.headers.get("Content-Length", "0"))
            try:
                body = json.loads(self.rfile.read(n) or b"{}")
                if self.path.split("?")[0].rstrip("/") in ("/v1/chat/completions", "/chat/completions", ""):
                    if body.get("stream"):
                        raise ValueError("streaming responses are not supported")
                    return self._reply(200, service.chat(body, self.headers.get("X-Session-Id")))
                self._reply(404, {"error": {"message": "unknown route", "type": "invalid_request_error"}})
            except Exception as e:  # noqa: BLE001
                self._reply(400, {"error": {"message": f"{type(e).__name__}: {e}", "type": "invalid_request_error"}})

    srv = ThreadingHTTPServer((host, port), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv, f"http://{host}:{srv.server_address[1]}"
