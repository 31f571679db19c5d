"""Hand file descriptors to other processes of the same node (``SCM_RIGHTS`` over a Unix socket).

A CUDA virtual-memory allocation is shared between processes by exporting it as a POSIX file descriptor
(``cuMemExportToShareableHandle``); the number itself means nothing in another process, the descriptor has to
travel as ancillary data of a Unix-domain socket message.  :class:`FdServer` runs in the owner of the memory and
answers every connection with ``(payload, fds)`` produced by a callback; :func:`fetch_fds` is the client side.
"""
from __future__ import annotations

import json
import os
import socket
import threading
from typing import Callable, List, Tuple


def socket_path(tag: str, rank: int) -> str:
    base = os.environ.get("RELAX_B200_SOCKET_DIR", "/tmp")
    return os.path.join(base, f"relax_b200_{tag}_{rank}.sock")


class FdServer:
    """Serves ``provider() -> (json-serialisable payload, [fd, ...])`` to every client that connects.  The provider
    is called per connection, so the descriptors can be exported fresh (and are closed here after sending)."""

    def __init__(self, path: str, provider: Callable[[], Tuple[dict, List[int]]], close_after_send: bool = True):
        self.path, self.provider, self.close_after_send = path, provider, close_after_send
        try:
            os.unlink(path)
        except FileNotFoundError:
            pass
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.sock.bind(path)
        self.sock.listen(64)
        self._stop = False
        self.served = 0
        self._t = threading.Thread(target=self._loop, daemon=True, name="fd-server")
        self._t.start()

    def _loop(self):
        while not self._stop:
            try:
                conn, _ = self.sock.accept()
            except OSError:
                return
            with conn:
                try:
                    payload, fds = self.provider()
                    msg = json.dumps(payload).encode()
                    socket.send_fds(conn, [len(msg).to_bytes(8, "little") + msg], list(fds))
                    self.served += 1
                    if self.close_after_send:
                        for fd in fds:
                            os.close(fd)
                except Exception as e:  # noqa: BLE001 - the client sees a closed connection and raises
                    try:
                        conn.sendall((0).to_bytes(8, "little"))
                    except OSError:
                        pass
                    self.last_error = repr(e)

    def close(self):
        self._stop = True
        try:
            self.sock.close()
        finally:
            try:
                os.unlink(self.path)
            except FileNotFoundError:
                pass


def fetch_fds(path: str, max_fds: int = 8, timeout: float = 60.0) -> Tuple[dict, List[int]]:
    """Connect to an :class:`FdServer` and return its ``(payload, fds)``; the caller owns the descriptors."""
    import time

    deadline = time.monotonic() + timeout
    while True:
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        try:
            s.connect(path)
            break
        except (FileNotFoundError, ConnectionRefusedError):
            s.close()
            if time.monotonic() > deadline:
                raise TimeoutError(f"no descriptor server at {path} after {timeout:.0f} s")
            time.sleep(0.05)
    with s:
        s.settimeout(timeout)
        data, fds, _flags, _addr = socket.recv_fds(s, 1 << 16, max_fds)
        if len(data) < 8:
            raise ConnectionError(f"descriptor server at {path} closed the connection")
        n = int.from_bytes(data[:8], "little")
        if n == 0:
            raise RuntimeError(f"descriptor server at {path} failed to produce its descriptors")
        body = data[8:]
        while len(body) < n:
            more = s.recv(n - len(body))
            if not more:
                raise ConnectionError("short read from the descriptor server")
            body += more
        return json.loads(body.decode()), list(fds)
