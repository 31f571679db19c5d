"""TransferQueue as a service: one process owns the queue, roles in other processes use it through a
TCP client with the same methods (plus ``async_*`` variants), as the reference's roles use the external
TransferQueue package through ``tq.get_client()`` (relax/utils/utils.py:508-556,
relax/utils/data/stream_dataloader.py:737-758, relax/components/advantages.py:96-112).

Wire format: 8-byte length + pickle of ``(method, args, kwargs)``; tensors travel as raw buffers next to
the pickle (no per-tensor pickling of storage).  On the receiving side tensors are materialised in
buffers drawn from a :class:`PinnedPool`, so a later ``.to(device, non_blocking=True)`` is a true
asynchronous copy and steady-state traffic allocates nothing.
"""
from __future__ import annotations

import asyncio
import io
import pickle
import socket
import socketserver
import struct
import threading
from typing import Dict, List, Optional, Tuple

import torch

from .transfer_queue import BatchMeta, TransferQueue

_METHODS = {"put", "seal", "get_meta", "get_data", "get_partition_list", "clear_partition", "reset_consumption",
            "check_production_status", "check_consumption_status", "check_stream_drained", "check_window_drained",
            "num_rows", "num_consumed"}


class PinnedPool:
    """Recycles page-locked host buffers by size class (powers of two)."""

    def __init__(self, pin: Optional[bool] = None, max_cached_bytes: int = 1 << 30):
        self.pin = torch.cuda.is_available() if pin is None else pin
        self.free: Dict[int, List[torch.Tensor]] = {}
        self.cached, self.max_cached = 0, max_cached_bytes
        self.allocations = self.reuses = 0
        self._lock = threading.Lock()

    @staticmethod
    def _cls(n: int) -> int:
        return 1 << max(9, (n - 1).bit_length())

    def take(self, nbytes: int) -> torch.Tensor:
        c = self._cls(nbytes)
        with self._lock:
            lst = self.free.get(c)
            if lst:
                self.cached -= c
                self.reuses += 1
                return lst.pop()
            self.allocations += 1
        return torch.empty(c, dtype=torch.uint8, pin_memory=self.pin)

    def give(self, buf: torch.Tensor):
        c = buf.numel()
        with self._lock:
            if self.cached + c <= self.max_cached:
                self.free.setdefault(c, []).append(buf)
                self.cached += c


# ----------------------------------------------------------------------------- framing
class _TensorRef:
    def __init__(self, idx, dtype, shape):
        self.idx, self.dtype, self.shape = idx, dtype, shape


def _encode(obj) -> Tuple[bytes, List[torch.Tensor]]:
    tensors: List[torch.Tensor] = []

    class P(pickle.Pickler):
        def persistent_id(self, o):
            if torch.is_tensor(o):
                t = o.detach().cpu().contiguous()
                tensors.append(t)
                return ("t", len(tensors) - 1, str(t.dtype), tuple(t.shape))
            return None

    bio = io.BytesIO()
    P(bio, protocol=pickle.HIGHEST_PROTOCOL).dump(obj)
    return bio.getvalue(), tensors


def _send(sock: socket.socket, obj):
    head, tensors = _encode(obj)
    sizes = [t.numel() * t.element_size() for t in tensors]
    sock.sendall(struct.pack("<QI", len(head), len(sizes)) + struct.pack(f"<{len(sizes)}Q", *sizes) + head)
    for t in tensors:
        if t.numel():
            sock.sendall(memoryview(t.view(torch.uint8).numpy()).cast("B") if t.dtype != torch.bfloat16
                         else memoryview(t.view(torch.uint8).numpy()).cast("B"))


def _recv_exact(sock: socket.socket, n: int, into: Optional[memoryview] = None) -> bytes:
    if into is not None:
        got = 0
        while got < n:
            r = sock.recv_into(into[got:n])
            if r == 0:
                raise ConnectionError("peer closed the connection")
            got += r
        return b""
    chunks, got = [], 0
    while got < n:
        c = sock.recv(min(1 << 20, n - got))
        if not c:
            raise ConnectionError("peer closed the connection")
        chunks.append(c)
        got += len(c)
    return b"".join(chunks)


def _recv(sock: socket.socket, pool: PinnedPool):
    hlen, nt = struct.unpack("<QI", _recv_exact(sock, 12))
    sizes = struct.unpack(f"<{nt}Q", _recv_exact(sock, 8 * nt)) if nt else ()
    head = _recv_exact(sock, hlen)
    bufs = []
    for s in sizes:
        b = pool.take(max(1, s))
        if s:
            _recv_exact(sock, s, memoryview(b.numpy())[:s])
        bufs.append(b)

    class U(pickle.Unpickler):
        def persistent_load(self, pid):
            _, idx, dtype, shape = pid
            dt = getattr(torch, dtype.replace("torch.", ""))
            n = 1
            for x in shape:
                n *= x
            nbytes = n * torch.empty(0, dtype=dt).element_size()
            return bufs[idx][:nbytes].view(dt).view(shape)

    return U(io.BytesIO(head)).load()


# ----------------------------------------------------------------------------- server / client
class TQServer:
    def __init__(self, queue: Optional[TransferQueue] = None, host: str = "127.0.0.1", port: int = 0):
        self.queue = queue or TransferQueue()
        pool = PinnedPool(pin=False)
        q = self.queue

        class Handler(socketserver.BaseRequestHandler):
            def handle(self):
                while True:
                    try:
                        method, args, kw = _recv(self.request, pool)
                    except (ConnectionError, struct.error, EOFError):
                        return
                    try:
                        if method not in _METHODS:
                            raise AttributeError(f"unknown method {method!r}")
                        out = ("ok", getattr(q, method)(*args, **kw))
                    except Exception as e:  # noqa: BLE001
                        out = ("err", f"{type(e).__name__}: {e}")
                    _send(self.request, out)

        class Srv(socketserver.ThreadingTCPServer):
            allow_reuse_address = True
            daemon_threads = True

        self.srv = Srv((host, port), Handler)
        self.address = self.srv.server_address
        threading.Thread(target=self.srv.serve_forever, daemon=True).start()

    def close(self):
        self.srv.shutdown()
        self.srv.server_close()


class TQClient:
    """Same calls as :class:`TransferQueue`; tensors of replies sit in pooled (pinned) host buffers."""

    def __init__(self, address, pool: Optional[PinnedPool] = None):
        self.sock = socket.create_connection(tuple(address))
        self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self.pool = pool or PinnedPool()
        self._lock = threading.Lock()

    def _call(self, method, *args, **kw):
        with self._lock:
            _send(self.sock, (method, args, kw))
            status, out = _recv(self.sock, self.pool)
        if status == "err":
            raise RuntimeError(out)
        return out

    def __getattr__(self, name):
        if name in _METHODS:
            return lambda *a, **k: self._call(name, *a, **k)
        if name.startswith("async_") and name[6:] in _METHODS:
            async def call(*a, **k):
                return await asyncio.get_running_loop().run_in_executor(None, lambda: self._call(name[6:], *a, **k))

            return call
        raise AttributeError(name)

    def close(self):
        try:
            self.sock.close()
        except OSError:
            pass
