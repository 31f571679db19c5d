"""OpenAPI 3 descriptions of the framework's HTTP surfaces (the reference's scripts/tools/generate_openapi.py):

    python -m relax_b200.utils.openapi --service metrics > metrics.openapi.json
    python -m relax_b200.utils.openapi --service all --out-dir api/

The route tables below are the single list of what each service answers; a test calls every listed route on a live
server, so the description cannot drift from the handlers.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, List, Tuple

_OBJ = {"type": "object"}

# service -> [(method, path, summary, request schema or None)]
ROUTES: Dict[str, List[Tuple[str, str, str, dict | None]]] = {
    "metrics": [
        ("get", "/health", "liveness", None),
        ("get", "/history", "every record logged so far", None),
        ("post", "/log_metric", "one scalar", {"type": "object", "required": ["step", "name", "value"],
                                               "properties": {"step": {"type": "integer"}, "name": {"type": "string"}, "value": {"type": "number"}}}),
        ("post", "/log_metrics_batch", "several scalars of one step", {"type": "object", "required": ["step", "metrics"],
                                                                       "properties": {"step": {"type": "integer"}, "metrics": _OBJ}}),
        ("post", "/report_step", "flush the step to the tracking adapters", {"type": "object", "required": ["step"],
                                                                             "properties": {"step": {"type": "integer"}}}),
        ("post", "/log_error", "an error record (forwarded to the notification adapters)", _OBJ),
    ],
    "coordinator": [
        ("get", "/health", "liveness", None),
        ("get", "/topology", "registered members by role and rank", None),
        ("post", "/register", "join with role, rank and address", _OBJ),
        ("post", "/unregister", "leave", _OBJ),
        ("post", "/heartbeat", "keep-alive of a member", _OBJ),
        ("post", "/global_rank", "global rank of (role, rank) in the weight-update world", _OBJ),
        ("post", "/get_model_update_group_ranks", "ranks and rendezvous of the per-pipeline-stage update groups", _OBJ),
        ("post", "/send_weight_meta", "publish the bucket layout of a weight version", _OBJ),
        ("post", "/recv_weight_meta", "long poll for the layout of the next weight version", _OBJ),
        ("post", "/clear_weight_meta", "drop published layouts", _OBJ),
    ],
    "chat": [
        ("get", "/health", "liveness", None),
        ("get", "/v1/models", "the served policy", None),
        ("post", "/v1/chat/completions", "OpenAI-compatible chat completion; `user` (or the X-Session-Id header) keys the session",
         {"type": "object", "required": ["messages"], "properties": {
             "messages": {"type": "array", "items": _OBJ}, "max_tokens": {"type": "integer"}, "n": {"type": "integer"},
             "logprobs": {"type": "boolean"}, "user": {"type": "string"}, "model": {"type": "string"}}}),
    ],
    "viewer": [
        ("get", "/", "index of dumped rollout steps (HTML)", None),
        ("get", "/step", "samples of one step (HTML); query: id, sort", None),
        ("get", "/sample", "one sample with per-token log-probs (HTML); query: id, n", None),
        ("get", "/api/steps", "per-step summaries (JSON)", None),
    ],
}


def build_spec(service: str, version: str = "0.1") -> dict:
    paths: dict = {}
    for method, path, summary, schema in ROUTES[service]:
        op = {"summary": summary, "responses": {"200": {"description": "ok"}, "400": {"description": "bad request"}}}
        if schema is not None:
            op["requestBody"] = {"required": True, "content": {"application/json": {"schema": schema}}}
        paths.setdefault(path, {})[method] = op
    return {"openapi": "3.0.3", "info": {"title": f"relax_b200 {service} service", "version": version}, "paths": paths}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--service", default="all", choices=["all"] + sorted(ROUTES))
    ap.add_argument("--out-dir", default=None)
    a = ap.parse_args(argv)
    names = sorted(ROUTES) if a.service == "all" else [a.service]
    for n in names:
        text = json.dumps(build_spec(n), indent=1)
        if a.out_dir:
            os.makedirs(a.out_dir, exist_ok=True)
            with open(os.path.join(a.out_dir, f"{n}.openapi.json"), "w") as f:
                f.write(text)
        else:
            print(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
