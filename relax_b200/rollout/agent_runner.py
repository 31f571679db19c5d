"""Agents as external commands: a launcher daemon, managed agent processes and their input / output contract.

An agent framework (a coding agent, a search agent, a gym client) runs as its own program: it is started once per
rollout session with a shell command, talks to the policy through the OpenAI-compatible endpoint of this package
(:mod:`relax_b200.rollout.openai_api`), and reports a reward when it exits.  The reference does the same with a
"managed command" (relax/agentic/runner/ipc.py: ``LauncherClient`` :148, ``SessionOutput`` :198,
``ManagedCommandAppSpec`` :297, ``ManagedAgentProcess`` :345, the session environment :432-442,
``ManagedAgentLauncher`` :521; flags ``--agent-command / --agent-cwd / --agent-env / --agent-timeout``,
relax/utils/arguments.py:1428-1465).

Contract with the agent process (environment variables):

``RELAX_BASE_URL``        the chat endpoint (``$RELAX_BASE_URL/v1/chat/completions``)
``RELAX_SESSION_ID``      send it as the ``X-Session-Id`` header (or ``user`` field): it ties the requests to the sample
``RELAX_GROUP_ID``        the prompt group of the sample, ``RELAX_ROLLOUT_MODE`` is ``train`` or ``eval``
``RELAX_INPUT_JSON``      a file with the sample's payload (prompt, label, metadata)
``RELAX_OUTPUT_JSON``     where the agent may write ``{"reward": number | object | null, "metadata": {...}}`` (or JSONL
                          records with ``name`` and ``messages``) before it exits with status 0
``RELAX_SESSION_IO_DIR``  a scratch directory that lives as long as the session

Why a daemon: the trainer process holds a CUDA context, pinned memory and many threads; ``fork`` from it is slow (page
tables of a very large process) and unsafe.  So ONE small helper process per node is started early
(``python -m relax_b200.rollout.agent_runner --socket PATH``) and every agent is its child.  One connection of the
Unix socket owns one agent: ``launch`` -> ``started`` -> ... -> ``exit``; ``terminate`` (or a closed connection) ends
the agent's whole process group, SIGTERM first and SIGKILL after a grace period.  Messages are JSON with a 4-byte
big-endian length prefix.

The time budget of an agent counts only while it is *active*: :meth:`ManagedAgent.set_active` pauses the clock while
the session waits at an admission gate, so a crowded engine does not time the agents out.
"""
from __future__ import annotations

import json
import os
import shutil
import signal
import socket
import struct
import subprocess
import sys
import tempfile
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Optional

_LEN = struct.Struct("!I")
GRACE_S = 5.0                     # between SIGTERM and SIGKILL of an agent's process group
BOOT_TIMEOUT_S = 30.0             # for the daemon to publish its socket


class AgentExecutionError(RuntimeError):
    """The agent failed (non-zero exit, timeout, unreadable output): its rollout group is dropped."""


# --------------------------------------------------------------------------- wire format
def _send(sock: socket.socket, obj: Mapping[str, Any]) -> None:
    body = json.dumps(obj, separators=(",", ":")).encode()
    sock.sendall(_LEN.pack(len(body)) + body)


def _recv_exact(sock: socket.socket, n: int) -> Optional[bytes]:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            return None
        buf += chunk
    return bytes(buf)


def _recv(sock: socket.socket) -> Optional[dict]:
    head = _recv_exact(sock, _LEN.size)
    if head is None:
        return None
    (n,) = _LEN.unpack(head)
    if n <= 0 or n > (64 << 20):
        raise ValueError(f"launcher message of {n} bytes")
    body = _recv_exact(sock, n)
    if body is None:
        return None
    obj = json.loads(body.decode())
    if not isinstance(obj, dict):
        raise ValueError("launcher message must be a JSON object")
    return obj


# --------------------------------------------------------------------------- agent output
@dataclass(frozen=True)
class SessionOutput:
    """What the agent wrote to ``RELAX_OUTPUT_JSON``: a reward and metadata for the recorded session, or explicit
    records (``name`` + ``messages`` each) that replace the recorded conversation."""
    metadata: dict = field(default_factory=dict)
    reward: Any = None
    records: tuple = ()

    @staticmethod
    def _check_reward(r):
        if r is not None and not isinstance(r, (int, float, dict)) or isinstance(r, bool):
            raise TypeError("'reward' must be null, a number or an object")

    @classmethod
    def from_text(cls, text: str) -> "SessionOutput":
        text = text.strip()
        if not text:
            return cls()
        try:
            obj = json.loads(text)
        except json.JSONDecodeError:
            obj = None
        if isinstance(obj, list):
            raise TypeError("explicit records are written one JSON object per line, not as an array")
        if isinstance(obj, dict) and "messages" not in obj:
            md = obj.get("metadata", {})
            if not isinstance(md, dict):
                raise TypeError("'metadata' must be an object")
            cls._check_reward(obj.get("reward"))
            return cls(metadata=md, reward=obj.get("reward"))
        rows = [obj] if isinstance(obj, dict) else [json.loads(line) for line in text.split("\n") if line.strip()]
        seen, recs = set(), []
        for r in rows:
            if not isinstance(r, dict) or "messages" not in r:
                raise TypeError("a record is an object with 'messages'")
            name = r.get("name")
            if not isinstance(name, str) or not name or name in seen:
                raise TypeError("every record needs a non-empty 'name', unique within the output")
            seen.add(name)
            msgs = r["messages"]
            if not isinstance(msgs, list) or not all(isinstance(m, dict) and "role" in m for m in msgs):
                raise TypeError("'messages' is a list of {role, content} objects")
            cls._check_reward(r.get("reward"))
            if not isinstance(r.get("metadata", {}), dict):
                raise TypeError("'metadata' must be an object")
            recs.append({k: r[k] for k in ("name", "messages", "metadata", "reward", "tools", "chat_template_kwargs") if k in r})
        return cls(records=tuple(recs))

    def scalar_reward(self) -> Optional[float]:
        """The number the trainer uses: the reward itself, or its ``reward`` / ``score`` entry when it is an object."""
        r = self.reward
        if isinstance(r, dict):
            r = r.get("reward", r.get("score"))
        return None if r is None else float(r)


@dataclass(frozen=True)
class AgentSpec:
    command: str
    cwd: str
    env: Mapping[str, str] = field(default_factory=dict)
    timeout_s: float = 1800.0

    def __post_init__(self):
        if not self.command.strip():
            raise ValueError("the agent command is empty")
        if not Path(self.cwd).is_dir():
            raise ValueError(f"the agent's working directory does not exist: {self.cwd}")
        if self.timeout_s <= 0:
            raise ValueError("the agent timeout must be positive")

    @classmethod
    def from_args(cls, args) -> "AgentSpec":
        env = {}
        for item in getattr(args, "agent_env", None) or []:
            if "=" not in item:
                raise ValueError(f"--agent-env {item!r}: expected KEY=VALUE")
            k, v = item.split("=", 1)
            env[k.strip()] = v
        if not getattr(args, "agent_command", None) or not getattr(args, "agent_cwd", None):
            raise ValueError("--use-agentic-rollout needs --agent-command and --agent-cwd")
        return cls(args.agent_command.strip(), str(Path(args.agent_cwd).expanduser().resolve()), env,
                   float(getattr(args, "agent_timeout", 1800.0) or 1800.0))


# --------------------------------------------------------------------------- the daemon (runs in its own small process)
def _kill_group(proc: subprocess.Popen, grace_s: float = GRACE_S) -> int:
    """SIGTERM the agent's process group, SIGKILL what is left after ``grace_s``; returns the exit status."""
    for sig, wait in ((signal.SIGTERM, grace_s), (signal.SIGKILL, grace_s)):
        if proc.poll() is not None:
            break
        try:
            os.killpg(proc.pid, sig)          # the agent was started as the leader of its own session
        except ProcessLookupError:
            break
        try:
            proc.wait(timeout=wait)
        except subprocess.TimeoutExpired:
            continue
    try:
        os.killpg(proc.pid, signal.SIGKILL)   # children that outlived the leader
    except (ProcessLookupError, PermissionError):
        pass
    return proc.poll() if proc.poll() is not None else -9


_LIVE: set = set()            # agent processes of this daemon that have not exited yet
_LIVE_LOCK = threading.Lock()


def _serve_connection(conn: socket.socket, grace_s: float) -> None:
    """One connection owns one agent process: launch, then wait for its exit or for a terminate request."""
    proc = None
    try:
        msg = _recv(conn)
        if msg is None:
            return                             # a liveness probe: connected and left
        if msg.get("op") != "launch":
            _send(conn, {"error": "expected a launch message"})
            return
        try:
            log = open(msg["log_path"], "ab", buffering=0)
            try:
                proc = subprocess.Popen(["/bin/sh", "-c", msg["command"]], cwd=msg["cwd"], env=dict(msg["env"]),
                                        stdin=subprocess.DEVNULL, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
            finally:
                log.close()
        except Exception as e:  # noqa: BLE001 - reported to the owner of the connection
            _send(conn, {"error": f"{type(e).__name__}: {e}"})
            return
        with _LIVE_LOCK:
            _LIVE.add(proc)
        _send(conn, {"op": "started", "pid": proc.pid})
        stop = threading.Event()

        def watch_owner():
            # a terminate message, or the owner going away, ends the agent
            try:
                while not stop.is_set():
                    m = _recv(conn)
                    if m is None or m.get("op") == "terminate":
                        break
            except (OSError, ValueError):
                pass
            if not stop.is_set():
                _kill_group(proc, grace_s)

        threading.Thread(target=watch_owner, daemon=True).start()
        code = proc.wait()
        stop.set()
        try:
            os.killpg(proc.pid, signal.SIGKILL)       # background children of a finished agent do not linger
        except (ProcessLookupError, PermissionError):
            pass
        try:
            _send(conn, {"op": "exit", "code": int(code)})
        except OSError:
            pass
    finally:
        if proc is not None and proc.poll() is None:
            _kill_group(proc, grace_s)
        with _LIVE_LOCK:
            _LIVE.discard(proc)
        try:
            conn.shutdown(socket.SHUT_RDWR)
        except OSError:
            pass
        conn.close()


def daemon_main(socket_path: str, grace_s: float = GRACE_S, parent_pid: Optional[int] = None) -> None:
    """Accept connections until the socket file is removed, the process that started the daemon is gone, or the
    daemon is signalled."""
    if os.path.exists(socket_path):
        os.unlink(socket_path)
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(socket_path)
    srv.listen(max(1024, socket.SOMAXCONN))
    srv.settimeout(0.5)
    try:
        while os.path.exists(socket_path):
            if parent_pid is not None and os.getppid() != parent_pid:
                break
            try:
                conn, _ = srv.accept()
            except socket.timeout:
                continue
            conn.settimeout(None)
            threading.Thread(target=_serve_connection, args=(conn, grace_s), daemon=True).start()
    finally:
        srv.close()
        try:
            os.unlink(socket_path)
        except FileNotFoundError:
            pass
        # the daemon leaves (its owner is gone or asked it to): no agent outlives it
        with _LIVE_LOCK:
            live = list(_LIVE)
        for proc in live:
            _kill_group(proc, min(grace_s, 1.0))


_DAEMONS: dict = {}
_DAEMON_LOCK = threading.Lock()


def ensure_launcher_daemon(socket_path: Optional[str] = None) -> str:
    """Start the node-local daemon once per process (idempotent) and return its socket path.  Call it early - before
    the CUDA context and the large allocations exist - so that the helper is forked from a small process."""
    with _DAEMON_LOCK:
        path = socket_path or os.path.join(tempfile.gettempdir(), f"relax_b200_launcher_{os.getpid()}.sock")
        p = _DAEMONS.get(path)
        if p is not None and p.poll() is None:
            return path
        root = str(Path(__file__).resolve().parents[2])
        env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        p = subprocess.Popen([sys.executable, "-m", "relax_b200.rollout.agent_runner", "--socket", path, "--parent", str(os.getpid())],
                             env=env, stdin=subprocess.DEVNULL, start_new_session=True)
        deadline = time.monotonic() + BOOT_TIMEOUT_S
        while True:
            if os.path.exists(path):
                try:
                    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
                        s.connect(path)
                    break
                except OSError:
                    pass
            if p.poll() is not None:
                raise RuntimeError(f"the launcher daemon exited with status {p.returncode}")
            if time.monotonic() > deadline:
                p.kill()
                raise TimeoutError("the launcher daemon did not come up")
            time.sleep(0.02)
        _DAEMONS[path] = p
        return path


def stop_launcher_daemon(socket_path: str) -> None:
    with _DAEMON_LOCK:
        p = _DAEMONS.pop(socket_path, None)
    try:
        os.unlink(socket_path)             # the accept loop sees it and leaves
    except FileNotFoundError:
        pass
    if p is not None:
        try:
            p.wait(timeout=3.0)
        except subprocess.TimeoutExpired:
            p.terminate()
            try:
                p.wait(timeout=3.0)
            except subprocess.TimeoutExpired:
                p.kill()


# --------------------------------------------------------------------------- client side: one managed agent
class ManagedAgent:
    """One agent process owned by one rollout session.

    ``start()`` writes the input file, asks the daemon to launch the command and returns; ``wait()`` blocks until the
    agent has exited and returns its :class:`SessionOutput` (or raises :class:`AgentExecutionError`).  The time budget
    runs only between ``set_active(True)`` and ``set_active(False)``."""

    def __init__(self, socket_path: str, spec: AgentSpec, session_id: str, group_id: str, payload: Mapping[str, Any],
                 base_url: str, rollout_mode: str = "train", keep_dir: bool = False):
        self.socket_path, self.spec, self.session_id, self.group_id = socket_path, spec, str(session_id), str(group_id)
        self.payload, self.base_url, self.rollout_mode, self.keep_dir = dict(payload), base_url, rollout_mode, keep_dir
        self.dir: Optional[str] = None
        self.pid: Optional[int] = None
        self._sock: Optional[socket.socket] = None
        self._lock = threading.Lock()
        self._remaining = float(spec.timeout_s)
        self._active_since: Optional[float] = None
        self._timer: Optional[threading.Timer] = None
        self._timed_out = self._terminated = False
        self._exit_code: Optional[int] = None
        self._exited = threading.Event()
        self.events: dict = {}

    # -- life cycle
    def start(self, active: bool = True) -> "ManagedAgent":
        self.dir = tempfile.mkdtemp(prefix="relax-b200-agent-")
        d = Path(self.dir)
        (d / "session_input.json").write_text(json.dumps(self.payload, separators=(",", ":"), ensure_ascii=False), encoding="utf-8")
        env = {**os.environ, **{str(k): str(v) for k, v in self.spec.env.items()},
               "RELAX_BASE_URL": self.base_url, "RELAX_SESSION_ID": self.session_id, "RELAX_ROLLOUT_MODE": self.rollout_mode,
               "RELAX_GROUP_ID": self.group_id, "RELAX_SESSION_IO_DIR": self.dir,
               "RELAX_INPUT_JSON": str(d / "session_input.json"), "RELAX_OUTPUT_JSON": str(d / "session_output.json")}
        self.events["launch_at"] = time.time()
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        try:
            s.connect(self.socket_path)
            _send(s, {"op": "launch", "command": self.spec.command, "cwd": self.spec.cwd, "env": env,
                      "log_path": str(d / "command.log"), "session_dir": self.dir})
            reply = _recv(s)
        except BaseException:
            s.close()
            self._cleanup()
            raise
        if reply is None or reply.get("op") != "started":
            s.close()
            self._cleanup()
            raise AgentExecutionError(f"the launcher did not start the agent: {(reply or {}).get('error', 'connection closed')}")
        self._sock, self.pid = s, reply.get("pid")
        self.events["started_at"] = time.time()
        threading.Thread(target=self._read_exit, daemon=True, name=f"agent-exit:{self.session_id}").start()
        if active:
            self.set_active(True)
        return self

    def _read_exit(self):
        try:
            while True:
                m = _recv(self._sock)
                if m is None:
                    break
                if m.get("op") == "exit":
                    self._exit_code = int(m.get("code", -1))
                    break
        except (OSError, ValueError):
            pass
        self.events["exit_at"] = time.time()
        self._exited.set()

    # -- the active-time budget
    def set_active(self, active: bool) -> None:
        with self._lock:
            if self._exited.is_set():
                return
            if active and self._active_since is None:
                self._active_since = time.monotonic()
                self._timer = threading.Timer(max(0.0, self._remaining), self._expire)
                self._timer.daemon = True
                self._timer.start()
            elif not active and self._active_since is not None:
                self._remaining -= time.monotonic() - self._active_since
                self._active_since = None
                if self._timer is not None:
                    self._timer.cancel()
                    self._timer = None

    @property
    def remaining_s(self) -> float:
        with self._lock:
            used = (time.monotonic() - self._active_since) if self._active_since is not None else 0.0
            return self._remaining - used

    def _expire(self):
        self._timed_out = True
        self._request_terminate()

    def _request_terminate(self):
        try:
            if self._sock is not None and not self._exited.is_set():
                _send(self._sock, {"op": "terminate"})
        except OSError:
            pass

    def terminate(self, join_s: float = 2 * GRACE_S + 1.0) -> None:
        """End the agent's process group (used when its group is dropped or the rollout is aborted)."""
        self._terminated = True
        self.set_active(False)
        self._request_terminate()
        self._exited.wait(join_s)
        self._close()

    # -- result
    def log_tail(self, limit: int = 8192) -> str:
        try:
            with open(os.path.join(self.dir, "command.log"), "rb") as f:
                f.seek(0, os.SEEK_END)
                n = f.tell()
                f.seek(max(0, n - limit))
                return f.read().decode("utf-8", errors="replace")
        except (OSError, TypeError):
            return ""

    def wait(self, poll_s: Optional[float] = None) -> SessionOutput:
        """Blocks until the agent is gone.  Raises :class:`AgentExecutionError` on a timeout, a non-zero status (unless
        the owner terminated it) or an unreadable output file."""
        self._exited.wait(poll_s)
        if not self._exited.is_set():
            raise TimeoutError("the agent is still running")
        self.set_active(False)
        try:
            tail = self.log_tail()
            if self._timed_out:
                raise AgentExecutionError(f"the agent timed out after {self.spec.timeout_s:g} s of active time\n{tail}".rstrip())
            if self._exit_code is None and not self._terminated:
                raise AgentExecutionError(f"the launcher connection was lost before the agent exited\n{tail}".rstrip())
            if self._exit_code not in (0, None) and not self._terminated:
                raise AgentExecutionError(f"the agent exited with status {self._exit_code}\n{tail}".rstrip())
            out = SessionOutput()
            path = os.path.join(self.dir, "session_output.json")
            if os.path.exists(path):
                try:
                    out = SessionOutput.from_text(Path(path).read_text(encoding="utf-8"))
                except Exception as e:  # noqa: BLE001
                    raise AgentExecutionError(f"the agent wrote an invalid output file: {e}\n{tail}".rstrip()) from e
            out.metadata.setdefault("agent_events", {}).update(self.events)
            return out
        finally:
            self._close()

    def _close(self):
        with self._lock:
            if self._timer is not None:
                self._timer.cancel()
                self._timer = None
        if self._sock is not None:
            try:
                self._sock.close()
            except OSError:
                pass
            self._sock = None
        self._cleanup()

    def _cleanup(self):
        if self.dir and not self.keep_dir:
            shutil.rmtree(self.dir, ignore_errors=True)


class AgentLauncher:
    """The command template bound to the node's daemon and to the chat endpoint the agents talk to."""

    def __init__(self, spec: AgentSpec, base_url: str, socket_path: Optional[str] = None):
        self.spec, self.base_url = spec, base_url.rstrip("/")
        self.socket_path = ensure_launcher_daemon(socket_path)

    def start_agent(self, session_id: str, group_id: str, payload: Mapping[str, Any], rollout_mode: str = "train",
                    active: bool = True) -> ManagedAgent:
        return ManagedAgent(self.socket_path, self.spec, session_id, group_id, payload, self.base_url, rollout_mode).start(active)

    def close(self):
        stop_launcher_daemon(self.socket_path)


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser("relax_b200 agent launcher daemon")
    ap.add_argument("--socket", required=True)
    ap.add_argument("--grace", type=float, default=GRACE_S)
    ap.add_argument("--parent", type=int, default=None, help="leave when this process is no longer the parent")
    a = ap.parse_args()
    daemon_main(a.socket, a.grace, a.parent)
