"""Rollout result dumps and their viewer: a JSONL file per rollout step, a small HTTP server that renders
them as HTML (index of steps -> table of samples -> one sample with per-token log-prob shading), and a plain-text
table for terminals.

Covers the reference's viewer (relax/utils/visualize/: ``server.py`` HTTP routes, ``templates.py`` pages,
``tui.py`` terminal view; relax/entrypoints/visualize.py launcher) and its ``--save-debug-rollout-data`` dump.
Only the standard library is used; pages are self-contained (no scripts or assets fetched from anywhere).

    python -m relax_b200.utils.visualize --dir dumps/ --port 8089        # browser
    python -m relax_b200.utils.visualize --dir dumps/ --text --step 3    # terminal
"""
from __future__ import annotations

import argparse
import html
import json
import os
import re
import statistics
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Callable, Dict, List, Optional, Sequence
from urllib.parse import parse_qs, urlparse

_FILE = re.compile(r"^rollout_(\d+)\.jsonl$")


# --------------------------------------------------------------------------- dump side
def _plain(v: Any):
    if hasattr(v, "tolist"):
        return v.tolist()
    if isinstance(v, dict):
        return {str(k): _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    if hasattr(v, "value") and not isinstance(v, (int, float, str, bool)):
        return v.value
    return v


def dump_rollout(directory: str, rollout_id: int, samples: Sequence[Any], decode: Optional[Callable[[list], str]] = None,
                 extra: Optional[Dict[str, Any]] = None) -> str:
    """Write ``rollout_<id>.jsonl``: a header line with step-level fields, then one line per sample.
    ``samples`` are :class:`relax_b200.types.Sample` objects or plain dicts."""
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, f"rollout_{int(rollout_id)}.jsonl")
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        f.write(json.dumps({"_header": True, "rollout_id": int(rollout_id), **_plain(extra or {})}) + "\n")
        for s in samples:
            d = s.to_dict() if hasattr(s, "to_dict") else dict(s)
            keep = {k: _plain(d.get(k)) for k in ("group_index", "index", "prompt", "response", "response_length", "reward",
                                                   "label", "status", "tokens", "loss_mask", "rollout_log_probs",
                                                   "weight_versions", "metadata") if d.get(k) is not None}
            if decode is not None and keep.get("tokens") and not keep.get("response"):
                R = int(keep.get("response_length") or 0)
                keep["response"] = decode(keep["tokens"][-R:]) if R else ""
                if not isinstance(keep.get("prompt"), str) or not keep["prompt"]:
                    keep["prompt"] = decode(keep["tokens"][:len(keep["tokens"]) - R])
            f.write(json.dumps(keep) + "\n")
    os.replace(tmp, path)
    return path


# --------------------------------------------------------------------------- read side
def list_steps(directory: str) -> List[int]:
    out = []
    for name in os.listdir(directory) if os.path.isdir(directory) else []:
        m = _FILE.match(name)
        if m:
            out.append(int(m.group(1)))
    return sorted(out)


def load_step(directory: str, rollout_id: int):
    header, samples = {}, []
    with open(os.path.join(directory, f"rollout_{int(rollout_id)}.jsonl")) as f:
        for line in f:
            if not line.strip():
                continue
            d = json.loads(line)
            if d.get("_header"):
                header = d
            else:
                samples.append(d)
    return header, samples


def _reward(s) -> Optional[float]:
    r = s.get("reward")
    if isinstance(r, dict):
        r = r.get("score", r.get("reward"))
    return float(r) if isinstance(r, (int, float)) else None


def step_summary(samples: Sequence[dict]) -> Dict[str, Any]:
    rs = [r for r in map(_reward, samples) if r is not None]
    ls = [int(s.get("response_length") or 0) for s in samples]
    groups: Dict[Any, list] = {}
    for s in samples:
        r = _reward(s)
        if r is not None:
            groups.setdefault(s.get("group_index"), []).append(r)
    flat = sum(1 for g in groups.values() if len(g) > 1 and max(g) == min(g))
    return {"samples": len(samples), "reward_mean": statistics.fmean(rs) if rs else None,
            "reward_std": statistics.pstdev(rs) if len(rs) > 1 else 0.0,
            "response_len_mean": statistics.fmean(ls) if ls else 0.0, "response_len_max": max(ls) if ls else 0,
            "truncated": sum(1 for s in samples if s.get("status") == "truncated"),
            "groups": len(groups), "zero_std_groups": flat}


# --------------------------------------------------------------------------- text view
def render_text(directory: str, rollout_id: Optional[int] = None, width: int = 60, limit: int = 50) -> str:
    steps = list_steps(directory)
    if not steps:
        return f"no rollout dumps under {directory}"
    if rollout_id is None:
        lines = [f"{'step':>6} {'samples':>8} {'reward':>9} {'std':>7} {'len':>8} {'trunc':>6} {'flat groups':>11}"]
        for st in steps:
            sm = step_summary(load_step(directory, st)[1])
            rm = "-" if sm["reward_mean"] is None else f"{sm['reward_mean']:.4f}"
            lines.append(f"{st:>6} {sm['samples']:>8} {rm:>9} {sm['reward_std']:>7.3f} {sm['response_len_mean']:>8.1f} "
                         f"{sm['truncated']:>6} {sm['zero_std_groups']:>5}/{sm['groups']:<5}")
        return "\n".join(lines)
    _, samples = load_step(directory, rollout_id)
    lines = [f"{'grp':>4} {'idx':>5} {'reward':>8} {'len':>6} {'status':>10}  response"]
    for s in samples[:limit]:
        r = _reward(s)
        txt = str(s.get("response", "")).replace("\n", "\\n")
        lines.append(f"{str(s.get('group_index', '-')):>4} {str(s.get('index', '-')):>5} "
                     f"{('-' if r is None else f'{r:.3f}'):>8} {int(s.get('response_length') or 0):>6} "
                     f"{str(s.get('status', '-')):>10}  {txt[:width]}")
    if len(samples) > limit:
        lines.append(f"... {len(samples) - limit} more")
    return "\n".join(lines)


# --------------------------------------------------------------------------- html view
_CSS = ("body{font:14px/1.4 sans-serif;margin:1.5em;color:#222}table{border-collapse:collapse}"
        "td,th{border:1px solid #ccc;padding:3px 8px;text-align:right}td.l{text-align:left;max-width:60em;"
        "overflow:hidden;white-space:nowrap;text-overflow:ellipsis}pre{white-space:pre-wrap;background:#f6f6f6;"
        "padding:8px}span.t{padding:1px 0}a{color:#06c;text-decoration:none}")


def _page(title: str, body: str) -> str:
    return f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(title)}</title><style>{_CSS}</style></head><body><h2>{html.escape(title)}</h2>{body}</body></html>"


def render_index(directory: str) -> str:
    rows = []
    for st in list_steps(directory):
        sm = step_summary(load_step(directory, st)[1])
        rm = "-" if sm["reward_mean"] is None else f"{sm['reward_mean']:.4f}"
        rows.append(f"<tr><td><a href='/step?id={st}'>{st}</a></td><td>{sm['samples']}</td><td>{rm}</td><td>{sm['reward_std']:.3f}</td>"
                    f"<td>{sm['response_len_mean']:.1f}</td><td>{sm['response_len_max']}</td><td>{sm['truncated']}</td>"
                    f"<td>{sm['zero_std_groups']}/{sm['groups']}</td></tr>")
    head = "<tr><th>step</th><th>samples</th><th>reward</th><th>std</th><th>mean len</th><th>max len</th><th>truncated</th><th>flat groups</th></tr>"
    return _page("Rollout steps", f"<table>{head}{''.join(rows)}</table>")


def render_step(directory: str, rollout_id: int, sort: str = "index") -> str:
    header, samples = load_step(directory, rollout_id)
    order = list(range(len(samples)))
    if sort == "reward":
        order.sort(key=lambda i: -(_reward(samples[i]) or 0.0))
    elif sort == "length":
        order.sort(key=lambda i: -int(samples[i].get("response_length") or 0))
    rows = []
    for i in order:
        s = samples[i]
        r = _reward(s)
        rows.append(f"<tr><td><a href='/sample?id={rollout_id}&n={i}'>{i}</a></td><td>{html.escape(str(s.get('group_index', '-')))}</td>"
                    f"<td>{'-' if r is None else f'{r:.3f}'}</td><td>{int(s.get('response_length') or 0)}</td>"
                    f"<td>{html.escape(str(s.get('status', '-')))}</td><td class='l'>{html.escape(str(s.get('response', ''))[:300])}</td></tr>")
    sm = step_summary(samples)
    info = html.escape(json.dumps({**{k: v for k, v in header.items() if k != '_header'}, **sm}))
    nav = f"<p><a href='/'>all steps</a> | sort: <a href='/step?id={rollout_id}&sort=index'>index</a> <a href='/step?id={rollout_id}&sort=reward'>reward</a> <a href='/step?id={rollout_id}&sort=length'>length</a></p>"
    head = "<tr><th>#</th><th>group</th><th>reward</th><th>len</th><th>status</th><th>response</th></tr>"
    return _page(f"Rollout {rollout_id}", f"{nav}<pre>{info}</pre><table>{head}{''.join(rows)}</table>")


def _shade(lp: float) -> str:
    """Background from white (log-prob 0) to red (log-prob <= -5)."""
    a = min(1.0, max(0.0, -lp / 5.0))
    return f"rgba(220,40,40,{a:.2f})"


def render_sample(directory: str, rollout_id: int, n: int, decode_token: Optional[Callable[[int], str]] = None) -> str:
    _, samples = load_step(directory, rollout_id)
    s = samples[n]
    body = [f"<p><a href='/step?id={rollout_id}'>back to rollout {rollout_id}</a></p>"]
    meta = {k: s.get(k) for k in ("group_index", "index", "reward", "label", "status", "response_length", "weight_versions", "metadata") if k in s}
    body.append(f"<pre>{html.escape(json.dumps(meta, indent=1))}</pre>")
    body.append(f"<h3>prompt</h3><pre>{html.escape(str(s.get('prompt', '')))}</pre>")
    body.append(f"<h3>response</h3><pre>{html.escape(str(s.get('response', '')))}</pre>")
    lps, toks = s.get("rollout_log_probs"), s.get("tokens")
    if lps and toks:
        R = len(lps)
        mask = s.get("loss_mask") or [1] * R
        spans = []
        for t, lp, m in zip(toks[-R:], lps, mask):
            txt = decode_token(t) if decode_token else str(t)
            style = f"background:{_shade(lp)}" + ("" if m else ";opacity:.45")
            spans.append(f"<span class='t' style='{style}' title='{lp:.3f}'>{html.escape(txt)}</span>")
        body.append("<h3>tokens (shaded by rollout log-prob; faded = masked out of the loss)</h3><p>" + " ".join(spans) + "</p>")
    return _page(f"Rollout {rollout_id} / sample {n}", "".join(body))


def make_server(directory: str, host: str = "127.0.0.1", port: int = 0, decode_token=None) -> ThreadingHTTPServer:
    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):   # quiet
            pass

        def do_GET(self):
            u = urlparse(self.path)
            q = {k: v[0] for k, v in parse_qs(u.query).items()}
            try:
                if u.path == "/":
                    body, ctype = render_index(directory), "text/html"
                elif u.path == "/step":
                    body, ctype = render_step(directory, int(q["id"]), q.get("sort", "index")), "text/html"
                elif u.path == "/sample":
                    body, ctype = render_sample(directory, int(q["id"]), int(q["n"]), decode_token), "text/html"
                elif u.path == "/api/steps":
                    body, ctype = json.dumps({st: step_summary(load_step(directory, st)[1]) for st in list_steps(directory)}), "application/json"
                else:
                    self.send_error(404)
                    return
            except (KeyError, ValueError, IndexError, FileNotFoundError) as e:
                self.send_error(400, str(e))
                return
            data = body.encode()
            self.send_response(200)
            self.send_header("Content-Type", ctype + "; charset=utf-8")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    return ThreadingHTTPServer((host, port), H)


def serve_in_thread(directory: str, host: str = "127.0.0.1", port: int = 0):
    srv = make_server(directory, host, port)
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    return srv, th


def main(argv=None):
    ap = argparse.ArgumentParser(description="Rollout result viewer")
    ap.add_argument("--dir", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8089)
    ap.add_argument("--text", action="store_true", help="print a table instead of serving HTML")
    ap.add_argument("--step", type=int, default=None)
    a = ap.parse_args(argv)
    if a.text:
        print(render_text(a.dir, a.step))
        return 0
    srv = make_server(a.dir, a.host, a.port)
    print(f"serving {a.dir} on http://{a.host}:{srv.server_address[1]}/")
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
