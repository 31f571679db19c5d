"""Distributed checkpoint service (DCS): the control plane and transport of weight updates between
roles that live in different processes (fully-async mode: actor -> actor_fwd / reference / rollout).

* :class:`TopologyManager` - who is registered (role, rank, address), heartbeats, global ranks of the
  weight-update world: actor ranks first, then actor_fwd, then reference, then one slot per rollout GPU
  (relax/distributed/checkpoint_service/coordinator/topology.py, service.py:375-411).
* :class:`Coordinator` - topology plus the weight-metadata mailbox: the sender posts
  ``(version, bucket layout)``, receivers long-poll for a version newer than the one they hold
  (service.py:413-450).  ``serve`` puts it behind HTTP routes for roles in other processes,
  :class:`CoordinatorClient` talks to either.
* :class:`TensorFusion` - packs many tensors into few flat buckets of bounded size with the metadata to
  unpack them (backends/base.py).
* :class:`DeviceDirectBackend` - sends the buckets with ``torch.distributed.broadcast`` over a dedicated
  process group (NCCL on GPUs, gloo in CPU tests) and, on the receiving side, allocates, receives and hands
  every tensor to ``load_weight`` (backends/device_direct.py:951-1077).
"""
from __future__ import annotations

import json
import threading
import time
import urllib.request
from dataclasses import dataclass, field
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

ROLE_ORDER = ("actor", "actor_fwd", "reference", "rollout")


@dataclass
class Member:
    role: str
    rank: int
    address: str = ""
    meta: dict = field(default_factory=dict)
    last_heartbeat: float = 0.0


class TopologyManager:
    def __init__(self, heartbeat_timeout_s: float = 120.0, clock: Callable[[], float] = time.monotonic):
        self.members: Dict[Tuple[str, int], Member] = {}
        self.timeout, self.clock = heartbeat_timeout_s, clock
        self._lock = threading.Lock()

    def register(self, role: str, rank: int, address: str = "", meta: Optional[dict] = None) -> int:
        if role not in ROLE_ORDER:
            raise ValueError(f"unknown role {role!r}")
        with self._lock:
            self.members[(role, rank)] = Member(role, rank, address, meta or {}, self.clock())
        return self.global_rank(role, rank)

    def unregister(self, role: str, rank: int):
        with self._lock:
            self.members.pop((role, rank), None)

    def heartbeat(self, role: str, rank: int) -> bool:
        with self._lock:
            m = self.members.get((role, rank))
            if m is None:
                return False
            m.last_heartbeat = self.clock()
            return True

    def alive(self, role: str, rank: int) -> bool:
        m = self.members.get((role, rank))
        return m is not None and self.clock() - m.last_heartbeat <= self.timeout

    def peers(self, role: str) -> List[Member]:
        with self._lock:
            return sorted((m for m in self.members.values() if m.role == role), key=lambda m: m.rank)

    def _ordered(self) -> List[Member]:
        return sorted(self.members.values(), key=lambda m: (ROLE_ORDER.index(m.role), m.rank))

    def global_rank(self, role: str, rank: int) -> int:
        with self._lock:
            for i, m in enumerate(self._ordered()):
                if (m.role, m.rank) == (role, rank):
                    return i
        raise KeyError((role, rank))

    def update_group_ranks(self, pp_size: int = 1) -> Dict[str, List[int]]:
        """One broadcast group per pipeline stage: the actor's TP-rank-0 of that stage sends to every
        forward-only / rollout member (``update_actor_pp_{stage}``)."""
        with self._lock:
            order = self._ordered()
        receivers = [i for i, m in enumerate(order) if m.role != "actor"]
        groups = {}
        for pp in range(pp_size):
            senders = [i for i, m in enumerate(order) if m.role == "actor" and m.meta.get("pp_rank", 0) == pp
                       and m.meta.get("tp_rank", 0) == 0 and m.meta.get("dp_rank", 0) == 0]
            if senders:
                groups[f"update_actor_pp_{pp}"] = [senders[0]] + receivers
        return groups

    def topology(self) -> dict:
        with self._lock:
            return {"members": [{"role": m.role, "rank": m.rank, "address": m.address, "meta": m.meta,
                                 "global_rank": i} for i, m in enumerate(self._ordered())]}


class Coordinator:
    def __init__(self, topology: Optional[TopologyManager] = None):
        self.topology = topology or TopologyManager()
        self._cv = threading.Condition()
        self._version = -1
        self._meta: Optional[dict] = None

    def send_weight_meta(self, version: int, meta: dict):
        with self._cv:
            if version <= self._version:
                raise ValueError(f"weight version must increase ({version} <= {self._version})")
            self._version, self._meta = version, meta
            self._cv.notify_all()

    def recv_weight_meta(self, last_version: int, timeout_s: float = 30.0) -> Optional[dict]:
        """Blocks until a version newer than ``last_version`` was posted; None on timeout."""
        with self._cv:
            if not self._cv.wait_for(lambda: self._version > last_version, timeout=timeout_s):
                return None
            return {"version": self._version, "meta": self._meta}

    def clear_weight_meta(self):
        with self._cv:
            self._meta = None

    def health(self) -> dict:
        return {"status": "ok", "members": len(self.topology.members), "weight_version": self._version}


class _Handler(BaseHTTPRequestHandler):
    coord: Coordinator = None

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
        c = self.coord
        if self.path == "/health":
            return self._reply(200, c.health())
        if self.path == "/topology":
            return self._reply(200, c.topology.topology())
        self._reply(404, {"error": "unknown route"})

    def do_POST(self):
        c = self.coord
        n = int(self.headers.get("Content-Length", "0"))
        try:
            b = json.loads(self.rfile.read(n) or b"{}")
            if self.path == "/register":
                out = {"global_rank": c.topology.register(b["role"], int(b["rank"]), b.get("address", ""), b.get("meta"))}
            elif self.path == "/unregister":
                c.topology.unregister(b["role"], int(b["rank"]))
                out = {"ok": True}
            elif self.path == "/heartbeat":
                out = {"ok": c.topology.heartbeat(b["role"], int(b["rank"]))}
            elif self.path == "/global_rank":
                out = {"global_rank": c.topology.global_rank(b["role"], int(b["rank"]))}
            elif self.path == "/get_model_update_group_ranks":
                out = c.topology.update_group_ranks(int(b.get("pp_size", 1)))
            elif self.path == "/send_weight_meta":
                c.send_weight_meta(int(b["version"]), b["meta"])
                out = {"ok": True}
            elif self.path == "/recv_weight_meta":
                out = c.recv_weight_meta(int(b.get("last_version", -1)), float(b.get("timeout_s", 30.0))) or {"version": None}
            elif self.path == "/clear_weight_meta":
                c.clear_weight_meta()
                out = {"ok": True}
            else:
                return self._reply(404, {"error": "unknown route"})
            self._reply(200, out)
        except Exception as e:  # noqa: BLE001
            self._reply(400, {"error": f"{type(e).__name__}: {e}"})


def serve(coord: Coordinator, host: str = "127.0.0.1", port: int = 0):
    srv = ThreadingHTTPServer((host, port), type("H", (_Handler,), {"coord": coord}))
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv, f"http://{host}:{srv.server_address[1]}"


class CoordinatorClient:
    def __init__(self, url: str, timeout_s: float = 60.0):
        self.url, self.timeout = url, timeout_s

    def _post(self, route, body, timeout=None):
        req = urllib.request.Request(self.url + route, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=timeout or self.timeout) as r:
            out = json.loads(r.read())
        if isinstance(out, dict) and "error" in out:
            raise RuntimeError(out["error"])
        return out

    def register(self, role, rank, address="", meta=None):
        return self._post("/register", {"role": role, "rank": rank, "address": address, "meta": meta or {}})["global_rank"]

    def unregister(self, role, rank):
        self._post("/unregister", {"role": role, "rank": rank})

    def heartbeat(self, role, rank):
        return self._post("/heartbeat", {"role": role, "rank": rank})["ok"]

    def update_group_ranks(self, pp_size=1):
        return self._post("/get_model_update_group_ranks", {"pp_size": pp_size})

    def send_weight_meta(self, version, meta):
        self._post("/send_weight_meta", {"version": version, "meta": meta})

    def recv_weight_meta(self, last_version, timeout_s=30.0):
        out = self._post("/recv_weight_meta", {"last_version": last_version, "timeout_s": timeout_s}, timeout=timeout_s + 10)
        return None if out.get("version") is None else out


# ----------------------------------------------------------------------------- tensors
@dataclass
class BucketLayout:
    dtype: str
    numel: int
    entries: List[Tuple[str, List[int], int]]   # (name, shape, offset)


class TensorFusion:
    """Greedy packing of named tensors into flat buckets of at most ``bucket_bytes`` (one dtype per bucket)."""

    def __init__(self, bucket_bytes: int = 512 << 20):
        self.bucket_bytes = bucket_bytes

    def plan(self, named: Iterable[Tuple[str, torch.Tensor]]) -> List[BucketLayout]:
        out: List[BucketLayout] = []
        cur: Dict[str, BucketLayout] = {}
        for name, t in named:
            key = str(t.dtype)
            lay = cur.get(key)
            nbytes = t.numel() * t.element_size()
            if lay is None or (lay.numel * t.element_size() + nbytes > self.bucket_bytes and lay.entries):
                lay = BucketLayout(key, 0, [])
                cur[key] = lay
                out.append(lay)
            lay.entries.append((name, list(t.shape), lay.numel))
            lay.numel += t.numel()
        return out

    @staticmethod
    def pack(layout: BucketLayout, tensors: Dict[str, torch.Tensor], device) -> torch.Tensor:
        dtype = getattr(torch, layout.dtype.replace("torch.", ""))
        buf = torch.empty(layout.numel, dtype=dtype, device=device)
        for name, shape, off in layout.entries:
            t = tensors[name]
            buf[off:off + t.numel()].copy_(t.reshape(-1))
        return buf

    @staticmethod
    def unpack(layout: BucketLayout, buf: torch.Tensor):
        for name, shape, off in layout.entries:
            n = 1
            for s in shape:
                n *= s
            yield name, buf[off:off + n].view(shape)


def _layout_to_json(l: BucketLayout) -> dict:
    return {"dtype": l.dtype, "numel": l.numel, "entries": l.entries}


def _layout_from_json(d: dict) -> BucketLayout:
    return BucketLayout(d["dtype"], int(d["numel"]), [(e[0], list(e[1]), int(e[2])) for e in d["entries"]])


class DeviceDirectBackend:
    """Bucketed broadcast of a weight version from ``src`` (a rank of ``group``) to all other ranks of it."""

    def __init__(self, coordinator, group=None, src: int = 0, bucket_bytes: int = 512 << 20, device="cpu"):
        self.coord, self.group, self.src, self.device = coordinator, group, src, torch.device(device)
        self.fusion = TensorFusion(bucket_bytes)
        self.version = -1

    def update_weights(self, named: Iterable[Tuple[str, torch.Tensor]], version: int) -> int:
        """Sender side: post the layout, then broadcast every bucket.  Returns the number of buckets."""
        named = list(named)
        plan = self.fusion.plan(named)
        self.coord.send_weight_meta(version, {"buckets": [_layout_to_json(l) for l in plan]})
        tensors = dict(named)
        for lay in plan:
            buf = self.fusion.pack(lay, tensors, self.device)
            dist.broadcast(buf, src=self.src, group=self.group)
        self.version = version
        return len(plan)

    def recv_weight(self, load_weight: Callable[[str, torch.Tensor], None], timeout_s: float = 60.0) -> Optional[int]:
        """Receiver side: wait for a newer version, receive its buckets, hand every tensor to ``load_weight``."""
        msg = self.coord.recv_weight_meta(self.version, timeout_s)
        if msg is None:
            return None
        for d in msg["meta"]["buckets"]:
            lay = _layout_from_json(d)
            dtype = getattr(torch, lay.dtype.replace("torch.", ""))
            buf = torch.empty(lay.numel, dtype=dtype, device=self.device)
            dist.broadcast(buf, src=self.src, group=self.group)
            for name, t in self.fusion.unpack(lay, buf):
                load_weight(name, t)
        self.version = msg["version"]
        return self.version
