"""On-policy distillation (OPD): a teacher scores the student's own samples and the per-token
divergence between the two is either folded into the advantages (as a dense reward) or added to the
policy loss.

Two token selections exist, as in the reference (relax/utils/opd/opd_utils.py:1097-1420):

* ``sampled_token`` - only the sampled token's log-prob under student and teacher is known (1-D);
  valid signals are ``reverse_kl`` (the single-sample estimate ``log p_s - log p_t``) and
  ``low_var_kl`` (the k3 estimator ``exp(-r) - 1 + r``);
* ``student_topk`` / ``teacher_topk`` / ``union`` - both distributions are known on a per-position
  set of K token ids (2-D, rows padded and masked for ``union``); the signal is a generalised
  Jensen-Shannon divergence with weight ``alpha`` on the teacher side (``alpha = 0`` reverse KL,
  ``alpha = 1`` forward KL), computed on the K ids plus - per ``norm_mode`` - a tail bin holding
  the remaining mass (``tail``), on the renormalised K ids (``norm``), or on the raw truncated
  ids (``trunc``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

KL_TYPES = ("reverse_kl", "forward_kl", "jsd", "low_var_kl")
TOKEN_SELECTIONS = ("sampled_token", "student_topk", "teacher_topk", "union")


def _prep(s, t, clamp, mask):
    s, t = s.float(), t.float()
    if clamp is not None:
        s, t = s.clamp_min(clamp), t.clamp_min(clamp)
    if mask is not None:
        s, t = s.masked_fill(~mask, -math.inf), t.masked_fill(~mask, -math.inf)
    return s, t


def _with_tail(lp):
    tot = torch.logsumexp(lp, -1, keepdim=True).clamp(max=-1e-7)
    return torch.cat([lp, torch.log(-torch.expm1(tot))], -1)


def _zero_pad(x, mask, k):
    return x if mask is None else x[..., :k].masked_fill(~mask, 0.0)


def token_kl(student_lp: torch.Tensor, teacher_lp: torch.Tensor, kl_type: str = "reverse_kl", alpha: float = 0.5,
             norm_mode: str = "tail", log_prob_min_clamp: Optional[float] = None,
             mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-position divergence.  1-D inputs ``[R]`` (sampled token) or 2-D ``[R, K]`` (log-probs on K ids per
    position, ``mask`` marks the valid columns of padded rows).  Returns ``[R]``."""
    if kl_type not in KL_TYPES:
        raise ValueError(f"unknown OPD divergence {kl_type!r}; one of {KL_TYPES}")
    s, t = _prep(student_lp, teacher_lp, log_prob_min_clamp, mask)
    if s.dim() == 1:
        r = s - t
        if kl_type == "reverse_kl":
            return r
        if kl_type == "low_var_kl":
            return torch.exp(-r) - 1.0 + r
        raise ValueError("with one sampled token per position only reverse_kl and low_var_kl are defined")
    k = s.shape[-1]
    if kl_type == "low_var_kl":
        r = s - t
        per = torch.exp(-r) - 1.0 + r
        if mask is not None:
            per = per.masked_fill(~mask, 0.0)
        return per.sum(-1)
    a = {"reverse_kl": 0.0, "forward_kl": 1.0}.get(kl_type, float(alpha))
    if not 0.0 <= a <= 1.0:
        raise ValueError("alpha must lie in [0, 1]")
    if norm_mode == "tail":
        s, t = _with_tail(s), _with_tail(t)
        if mask is not None:   # the tail bin is always valid
            mask = torch.cat([mask, torch.ones_like(mask[..., :1])], -1)
            k += 1
    elif norm_mode == "norm":
        s, t = s - torch.logsumexp(s, -1, keepdim=True), t - torch.logsumexp(t, -1, keepdim=True)
    elif norm_mode != "trunc":
        raise ValueError("norm_mode is tail, norm or trunc")

    def kl(p, q):   # sum_i exp(p_i) (p_i - q_i), padded columns contribute nothing
        term = p.exp() * (p - q)
        term = torch.where(torch.isfinite(p), term, torch.zeros_like(term))
        return _zero_pad(term, mask, k).sum(-1)

    if a == 0.0:
        return kl(s, t)
    if a == 1.0:
        return kl(t, s)
    m = torch.logsumexp(torch.stack([s + math.log(1.0 - a), t + math.log(a)]), 0)
    return (1.0 - a) * kl(s, m) + a * kl(t, m)


def union_ids(student_ids: torch.Tensor, teacher_ids: torch.Tensor):
    """Row-wise union of two ``[R, K]`` id sets: ``(ids [R, K'], lengths [R])`` padded with the row's first id."""
    R = student_ids.shape[0]
    both = torch.cat([student_ids, teacher_ids], -1)
    srt, _ = both.sort(-1)
    keep = torch.ones_like(srt, dtype=torch.bool)
    keep[:, 1:] = srt[:, 1:] != srt[:, :-1]
    lengths = keep.sum(-1)
    kmax = int(lengths.max()) if R else 0
    out = srt[:, :1].expand(R, kmax).clone()
    pos = keep.cumsum(-1) - 1
    rows = torch.arange(R, device=srt.device)[:, None].expand_as(srt)
    out[rows[keep], pos[keep]] = srt[keep]
    return out, lengths


def per_token_signal(selection: str, *, student_lp=None, teacher_lp=None, student_topk_lp=None, teacher_topk_lp=None,
                     k_lengths=None, **kw) -> torch.Tensor:
    if selection not in TOKEN_SELECTIONS:
        raise ValueError(f"unknown token selection {selection!r}")
    if selection == "sampled_token":
        return token_kl(student_lp, teacher_lp, **kw)
    mask = None
    if selection == "union" and k_lengths is not None:
        mask = torch.arange(teacher_topk_lp.shape[-1], device=teacher_topk_lp.device)[None, :] < k_lengths[:, None]
    return token_kl(student_topk_lp, teacher_topk_lp, mask=mask, **kw)


def apply_to_advantages(advantages: List[torch.Tensor], signals: Sequence[torch.Tensor], coef: float,
                        per_token_clip: Optional[float] = None) -> List[torch.Tensor]:
    """``A_t <- A_t - coef * D_t``: the divergence acts as a per-token penalty (a dense reward of ``-D_t``)."""
    if coef == 0.0:
        return advantages
    out = []
    for a, d in zip(advantages, signals):
        d = d.detach().to(a.device)
        if per_token_clip is not None:
            d = d.clamp(max=float(per_token_clip))
        out.append(a - coef * d)
    return out


def opd_loss(signals: torch.Tensor, loss_masks: Sequence[torch.Tensor], response_lengths: Sequence[int],
             coef: float) -> torch.Tensor:
    """Masked token mean of the (differentiable) divergence over a packed batch, times ``coef``."""
    chunks = torch.split(signals, list(response_lengths))
    num = sum((c * m.to(c)).sum() for c, m in zip(chunks, loss_masks))
    den = sum(m.sum() for m in loss_masks)
    return coef * num / torch.clamp_min(torch.as_tensor(den, dtype=signals.dtype, device=signals.device), 1)


class InProcessTeacher:
    """Teacher scoring through a forward-only :class:`~relax_b200.train.actor.TrainActor` (or its ``teacher``
    weight snapshot): the managed-teacher role of the reference (relax/distributed/ray/teacher_manager.py)
    reduced to the call the pipeline needs."""

    def __init__(self, actor, tag: str = "actor"):
        self.actor, self.tag = actor, tag

    def score(self, batch: dict) -> List[torch.Tensor]:
        return self.actor.compute_log_prob(batch, self.tag)["log_probs"]


class HTTPTeacher:
    """A teacher behind ``POST <url>/score`` (``{"tokens": [[...]], "response_lengths": [...]}`` ->
    ``{"log_probs": [[...]]}``): what ``--opd-teacher-urls`` names (the reference scores against teacher engines
    over HTTP, relax/engine/rollout/on_policy_distillation.py).  :func:`serve_teacher` is the matching server."""

    def __init__(self, url: str, timeout_s: float = 600.0):
        self.url, self.timeout_s = url.rstrip("/"), timeout_s

    def score(self, batch: dict) -> List[torch.Tensor]:
        import json
        import urllib.request

        body = json.dumps({"tokens": [[int(t) for t in x] for x in batch["tokens"]],
                           "response_lengths": [int(r) for r in batch["response_lengths"]]}).encode()
        req = urllib.request.Request(self.url + "/score", data=body, headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
            out = json.loads(r.read().decode())
        return [torch.tensor(x, dtype=torch.float32) for x in out["log_probs"]]


def serve_teacher(scorer, host: str = "127.0.0.1", port: int = 0):
    """Serve ``scorer.score(batch)`` (an :class:`InProcessTeacher`, anything with that call) over HTTP in a daemon
    thread: ``POST /score`` and ``GET /health``.  Returns ``(server, thread)``; one request is scored at a time
    (the scorer owns a GPU)."""
    import json
    import threading
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    lock = threading.Lock()

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):       # quiet
            pass

        def _send(self, code, obj):
            data = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def do_GET(self):
            self._send(200, {"status": "ok"}) if self.path.rstrip("/") == "/health" else self._send(404, {"error": "not found"})

        def do_POST(self):
            if self.path.rstrip("/") != "/score":
                return self._send(404, {"error": "not found"})
            try:
                req = json.loads(self.rfile.read(int(self.headers.get("Content-Length", "0"))).decode())
                with lock:
                    lp = scorer.score({"tokens": req["tokens"], "response_lengths": req["response_lengths"]})
                self._send(200, {"log_probs": [[float(v) for v in x.tolist()] for x in lp]})
            except Exception as e:   # noqa: BLE001 - the client marks this teacher unhealthy and retries elsewhere
                self._send(500, {"error": repr(e)})

    srv = ThreadingHTTPServer((host, port), H)
    t = threading.Thread(target=srv.serve_forever, daemon=True, name="teacher-server")
    t.start()
    return srv, t


class TeacherPool:
    """Several teacher scorers behind one ``score`` call: the batch is cut into per-teacher slices that run
    concurrently, a teacher that raises or exceeds the time limit is marked unhealthy and its slice is re-run on
    the next healthy one, and unhealthy teachers are retried after ``retry_after_s`` (the managed teacher engines of
    relax/distributed/ray/teacher_manager.py: start, health, pick, recover).  A teacher is any object with
    ``score(batch) -> list`` (:class:`InProcessTeacher`, a remote scorer, a rollout engine in scoring mode)."""

    def __init__(self, teachers: Sequence, timeout_s: float = 600.0, retry_after_s: float = 60.0):
        if not teachers:
            raise ValueError("TeacherPool needs at least one teacher")
        self.teachers = list(teachers)
        self.timeout_s, self.retry_after_s = timeout_s, retry_after_s
        self._down: dict = {}          # index -> time it was marked unhealthy
        self.failures = 0

    def healthy(self) -> List[int]:
        import time

        now = time.monotonic()
        for i, t0 in list(self._down.items()):
            if now - t0 >= self.retry_after_s:
                del self._down[i]
        return [i for i in range(len(self.teachers)) if i not in self._down]

    @staticmethod
    def _slice(batch: dict, idx: Sequence[int]) -> dict:
        n = len(batch["tokens"])
        return {k: ([v[i] for i in idx] if isinstance(v, (list, tuple)) and len(v) == n else v) for k, v in batch.items()}

    def score(self, batch: dict) -> List[torch.Tensor]:
        import time
        from concurrent.futures import ThreadPoolExecutor, TimeoutError as _Timeout

        n = len(batch["tokens"])
        out: List = [None] * n
        pending = list(range(n))
        while pending:
            live = self.healthy()
            if not live:
                raise RuntimeError("no healthy teacher left")
            parts = [pending[j::len(live)] for j in range(len(live))]
            jobs = [(t, p) for t, p in zip(live, parts) if p]
            retry: List[int] = []
            with ThreadPoolExecutor(max_workers=len(jobs)) as ex:
                futs = [(t, p, ex.submit(self.teachers[t].score, self._slice(batch, p))) for t, p in jobs]
                for t, p, f in futs:
                    try:
                        res = f.result(timeout=self.timeout_s)
                        if len(res) != len(p):
                            raise RuntimeError(f"teacher {t} returned {len(res)} rows for {len(p)} samples")
                        for i, r in zip(p, res):
                            out[i] = r
                    except (_Timeout, Exception):   # noqa: BLE001 - any failure of a teacher is handled the same way
                        self._down[t] = time.monotonic()
                        self.failures += 1
                        retry.extend(p)
            pending = sorted(retry)
        return out
