"""Trajectory replay: record the exact inputs and outputs of the numerically delicate stages of a
training step (reward post-processing, advantage estimation, the policy loss) and re-run them
offline, to bisect a regression or reproduce a divergence without the cluster
(relax/utils/replay/: capture hooks in the loss / advantage / reward stages, bundle, offline runner).

A bundle is a directory: ``manifest.json`` lists the captured records; each record is one ``.pt``
file holding ``{"inputs": {...}, "outputs": {...}}`` with tensors moved to the CPU.

What makes a bundle self-describing and checkable (relax/utils/replay/{identity,schema,validate,selection,report}.py):

* *identity*: the manifest names the run (model, loss configuration hash, world layout and this rank's place in it,
  dtype, library versions); :func:`validate_bundle` refuses to mix records of different identities.
* *integrity*: every record carries the SHA-256 of its file; a ``COMPLETE`` marker is written when the recorder is
  closed, with the number of records - a bundle of a crashed run is recognisable.
* *selection*: replay a subset - stages, rollout ids, optimizer steps - with :func:`select_records`.
* *report*: :func:`first_divergence` orders the results by (rollout, step, stage order) and names the first record,
  field and size of the first difference; ``python -m relax_b200.utils.replay inspect | validate | replay <bundle>``.

Capture in a training run is switched on by the environment (relax/utils/replay/capture.py:521-560):
``RELAX_REPLAY_CAPTURE_DIR`` (one sub-directory per rank), ``RELAX_REPLAY_CAPTURE_ROLLOUTS`` (``id,id,...``; default:
all), ``RELAX_REPLAY_CAPTURE_STEPS`` (``rollout:step,...``), ``RELAX_REPLAY_CAPTURE_MAX`` (records per rank, 64).
Records are written by a background thread; the training step only pays for the copy of the tensors to the host.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import queue
import threading
import time
from typing import Callable, Dict, Iterable, Optional

import torch

STAGES = ("reward", "advantages", "loss")         # in the order a training step runs them


def _to_cpu(x):
    if torch.is_tensor(x):
        return x.detach().cpu()
    if dataclasses.is_dataclass(x) and not isinstance(x, type):
        return {"__dataclass__": type(x).__module__ + ":" + type(x).__qualname__,
                "fields": {f.name: _to_cpu(getattr(x, f.name)) for f in dataclasses.fields(x)}}
    if isinstance(x, dict):
        return {k: _to_cpu(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_to_cpu(v) for v in x)
    return x


def _restore(x):
    if isinstance(x, dict) and "__dataclass__" in x:
        import importlib

        mod, _, qual = x["__dataclass__"].partition(":")
        cls = importlib.import_module(mod)
        for part in qual.split("."):
            cls = getattr(cls, part)
        return cls(**{k: _restore(v) for k, v in x["fields"].items()})
    if isinstance(x, dict):
        return {k: _restore(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_restore(v) for v in x)
    return x


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def run_identity(model: str = "", config=None, layout: Optional[dict] = None, dtype: str = "") -> dict:
    """What a record belongs to: the model, a hash of the (loss) configuration, the parallel layout and versions."""
    cfg_text = ""
    if config is not None:
        d = dataclasses.asdict(config) if dataclasses.is_dataclass(config) else dict(config)
        cfg_text = json.dumps({k: (v if isinstance(v, (int, float, str, bool, type(None))) else str(v)) for k, v in sorted(d.items())})
    return {"model": model, "config_sha": hashlib.sha256(cfg_text.encode()).hexdigest()[:16], "layout": dict(layout or {}),
            "dtype": dtype, "torch": torch.__version__, "format": 2}


class ReplayRecorder:
    def __init__(self, out_dir: Optional[str], stages: Iterable[str] = STAGES, max_records: int = 64, rank: int = 0,
                 identity: Optional[dict] = None, rollouts: Optional[Iterable[int]] = None, steps: Optional[Iterable[tuple]] = None,
                 background: bool = False):
        self.out_dir, self.stages, self.max_records, self.rank = out_dir, set(stages), max_records, rank
        self.identity = identity or run_identity()
        self.rollouts = None if rollouts is None else set(int(r) for r in rollouts)
        self.steps = None if steps is None else set((int(r), int(s_)) for r, s_ in steps)
        self.records: list = []
        self._lock = threading.Lock()
        self._q: Optional[queue.Queue] = None
        self._thread = None
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)
            if background:
                self._q = queue.Queue()
                self._thread = threading.Thread(target=self._writer, daemon=True, name="replay-capture-writer")
                self._thread.start()

    @classmethod
    def from_env(cls, rank: int = 0, identity: Optional[dict] = None) -> "ReplayRecorder":
        """The recorder a training process uses: off unless ``RELAX_REPLAY_CAPTURE_DIR`` is set."""
        root = os.environ.get("RELAX_REPLAY_CAPTURE_DIR")
        if not root:
            return cls(None)
        ro = os.environ.get("RELAX_REPLAY_CAPTURE_ROLLOUTS")
        st = os.environ.get("RELAX_REPLAY_CAPTURE_STEPS")
        try:
            rollouts = [int(x) for x in ro.split(",") if x.strip()] if ro else None
            steps = [tuple(int(y) for y in x.split(":")) for x in st.split(",") if x.strip()] if st else None
            if steps is not None and any(len(t) != 2 for t in steps):
                raise ValueError
        except ValueError:
            raise ValueError("RELAX_REPLAY_CAPTURE_ROLLOUTS is 'id,id,...' and RELAX_REPLAY_CAPTURE_STEPS 'rollout:step,...'") from None
        rec = cls(os.path.join(root, f"rank-{rank}"), max_records=int(os.environ.get("RELAX_REPLAY_CAPTURE_MAX", "64")), rank=rank,
                  identity=identity, rollouts=rollouts, steps=steps, background=True)
        import atexit

        atexit.register(rec.close)            # a run that ends normally leaves a complete bundle behind
        return rec

    @property
    def enabled(self) -> bool:
        return self.out_dir is not None

    def wants(self, stage: str, rollout_id: int, step_id: Optional[int] = None) -> bool:
        """Cheap test before the caller assembles the inputs."""
        if not self.enabled or stage not in self.stages or len(self.records) >= self.max_records:
            return False
        if self.steps is not None and step_id is not None:
            return (int(rollout_id), int(step_id)) in self.steps
        if self.steps is not None and step_id is None:
            return any(r == int(rollout_id) for r, _ in self.steps)
        return self.rollouts is None or int(rollout_id) in self.rollouts

    def capture(self, stage: str, rollout_id: int, inputs: dict, outputs, step_id: Optional[int] = None) -> Optional[str]:
        if not self.wants(stage, rollout_id, step_id):
            return None
        with self._lock:
            name = f"{stage}_r{rollout_id}" + (f"_s{step_id}" if step_id is not None else "") + f"_rank{self.rank}_{len(self.records):04d}.pt"
            rec = {"stage": stage, "rollout_id": int(rollout_id), "step_id": step_id, "file": name, "time": time.time(), "sha256": None}
            self.records.append(rec)
        blob = {"inputs": _to_cpu(inputs), "outputs": _to_cpu(outputs)}       # the copy to the host happens here, on the caller
        if self._q is not None:
            self._q.put((rec, blob))
        else:
            self._write(rec, blob)
        return name

    def _write(self, rec, blob):
        path = os.path.join(self.out_dir, rec["file"])
        torch.save(blob, path)
        rec["sha256"] = _sha256(path)
        with self._lock:
            with open(os.path.join(self.out_dir, "manifest.json"), "w") as f:
                json.dump({"identity": self.identity, "rank": self.rank, "records": [r for r in self.records if r["sha256"]]}, f, indent=1)

    def _writer(self):
        while True:
            item = self._q.get()
            if item is None:
                return
            try:
                self._write(*item)
            except Exception:  # noqa: BLE001 - a failed capture must not take the training run down
                pass

    def close(self):
        """Flush the writer and mark the bundle complete (safe to call twice)."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        if self._q is not None:
            self._q.put(None)
            self._thread.join(timeout=60)
            self._q = None
        if self.enabled:
            with open(os.path.join(self.out_dir, "COMPLETE"), "w") as f:
                json.dump({"records": len([r for r in self.records if r["sha256"]]), "rank": self.rank}, f)

    def wrap(self, stage: str, fn: Callable, rollout_id_fn: Callable[[], int] = lambda: -1) -> Callable:
        """``fn(**kwargs)`` recorded transparently."""
        def inner(**kw):
            out = fn(**kw)
            self.capture(stage, rollout_id_fn(), kw, out)
            return out

        return inner


def _compare(a, b, atol, rtol, path, diffs):
    if torch.is_tensor(a) and torch.is_tensor(b):
        if a.shape != b.shape:
            diffs.append((path, f"shape {tuple(a.shape)} vs {tuple(b.shape)}"))
        elif not torch.allclose(a.float(), b.float(), atol=atol, rtol=rtol, equal_nan=True):
            diffs.append((path, f"max abs diff {float((a.float() - b.float()).abs().max()):.3e}"))
    elif isinstance(a, dict) and isinstance(b, dict):
        for k in a:
            if k in b:
                _compare(a[k], b[k], atol, rtol, f"{path}.{k}", diffs)
            else:
                diffs.append((f"{path}.{k}", "missing in replay"))
    elif isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)):
        if len(a) != len(b):
            diffs.append((path, f"length {len(a)} vs {len(b)}"))
        for i, (x, y) in enumerate(zip(a, b)):
            _compare(x, y, atol, rtol, f"{path}[{i}]", diffs)
    elif isinstance(a, float) and isinstance(b, float):
        if abs(a - b) > atol + rtol * abs(a):
            diffs.append((path, f"{a} vs {b}"))


def default_stage_functions() -> Dict[str, Callable]:
    from ..algo import loss as L
    from ..algo.ppo_utils import post_process_rewards

    def run_loss(log_probs, entropy, batch, cfg):
        loss, metrics = L.policy_loss(log_probs, entropy, batch, cfg)
        return {"loss": loss, "metrics": metrics}

    def run_adv(**kw):
        adv, ret = L.compute_advantages_and_returns(**kw)
        return {"advantages": adv, "returns": ret}

    return {"loss": run_loss, "advantages": run_adv, "reward": lambda **kw: post_process_rewards(**kw)}


def load_manifest(bundle_dir: str) -> dict:
    """The manifest of a rank-local bundle, or - for a directory of ``rank-*`` bundles - all of them merged (records
    get a ``dir`` entry)."""
    path = os.path.join(bundle_dir, "manifest.json")
    if os.path.exists(path):
        m = json.load(open(path))
        for r in m["records"]:
            r.setdefault("dir", bundle_dir)
        m.setdefault("identity", {})
        return m
    subs = sorted(d for d in os.listdir(bundle_dir) if d.startswith("rank-") and os.path.isdir(os.path.join(bundle_dir, d)))
    if not subs:
        raise FileNotFoundError(f"{bundle_dir}: no manifest.json and no rank-* bundles")
    parts = [load_manifest(os.path.join(bundle_dir, d)) for d in subs]
    return {"identity": parts[0].get("identity", {}), "ranks": [p.get("rank") for p in parts],
            "identities": [p.get("identity", {}) for p in parts], "records": [r for p in parts for r in p["records"]]}


def select_records(records: list, stages: Optional[Iterable[str]] = None, rollouts: Optional[Iterable[int]] = None,
                   steps: Optional[Iterable[tuple]] = None) -> list:
    """The records of the chosen stages / rollout ids / (rollout, step) pairs, in the order a run produces them."""
    st = None if stages is None else set(stages)
    ro = None if rollouts is None else set(int(x) for x in rollouts)
    sp = None if steps is None else set((int(a_), int(b_)) for a_, b_ in steps)
    out = [r for r in records if (st is None or r["stage"] in st) and (ro is None or r["rollout_id"] in ro)
           and (sp is None or r.get("step_id") is None or (r["rollout_id"], r["step_id"]) in sp)]
    order = {n: i for i, n in enumerate(STAGES)}
    return sorted(out, key=lambda r: (r["rollout_id"], -1 if r.get("step_id") is None else r["step_id"], order.get(r["stage"], 99), r["file"]))


def validate_bundle(bundle_dir: str) -> list:
    """Format, integrity and consistency, without running anything: a list of problems (empty = valid)."""
    problems = []
    try:
        m = load_manifest(bundle_dir)
    except (OSError, ValueError) as e:
        return [f"manifest: {e}"]
    ids = m.get("identities") or [m.get("identity", {})]
    strip = lambda d: {k: v for k, v in d.items() if k != "layout"}
    if any(strip(i) != strip(ids[0]) for i in ids):
        problems.append("the rank bundles come from different runs (model / configuration / versions differ)")
    dirs = sorted({r["dir"] for r in m["records"]}) or [bundle_dir]
    for d in dirs:
        mark = os.path.join(d, "COMPLETE")
        if not os.path.exists(mark):
            problems.append(f"{d}: no COMPLETE marker (the run did not close the recorder)")
        else:
            n = json.load(open(mark)).get("records")
            have = len([r for r in m["records"] if r["dir"] == d])
            if n != have:
                problems.append(f"{d}: COMPLETE counts {n} records, the manifest lists {have}")
    for r in m["records"]:
        path = os.path.join(r["dir"], r["file"])
        if r["stage"] not in STAGES:
            problems.append(f"{r['file']}: unknown stage {r['stage']!r}")
        if not os.path.exists(path):
            problems.append(f"{r['file']}: file is missing")
        elif r.get("sha256") and _sha256(path) != r["sha256"]:
            problems.append(f"{r['file']}: checksum differs (the file changed after capture)")
    return problems


def replay_bundle(bundle_dir: str, stage_fns: Optional[Dict[str, Callable]] = None, atol: float = 1e-6,
                  rtol: float = 1e-5, stages: Optional[Iterable[str]] = None, rollouts: Optional[Iterable[int]] = None,
                  steps: Optional[Iterable[tuple]] = None) -> list:
    """Re-run the (selected) records of a bundle through ``stage_fns[stage](**inputs)``; returns one report per record,
    in run order: ``{"file", "stage", "rollout_id", "step_id", "ok", "diffs": [(where, what), ...]}``."""
    fns = stage_fns or default_stage_functions()
    manifest = load_manifest(bundle_dir)
    reports = []
    for rec in select_records(manifest["records"], stages, rollouts, steps):
        blob = torch.load(os.path.join(rec.get("dir", bundle_dir), rec["file"]), weights_only=False)
        fn = fns.get(rec["stage"])
        base = {"file": rec["file"], "stage": rec["stage"], "rollout_id": rec["rollout_id"], "step_id": rec.get("step_id")}
        if fn is None:
            reports.append(dict(base, ok=None, diffs=[("", "no function for this stage")]))
            continue
        out = _to_cpu(fn(**_restore(blob["inputs"])))
        diffs: list = []
        _compare(blob["outputs"], out, atol, rtol, "out", diffs)
        reports.append(dict(base, ok=not diffs, diffs=diffs))
    return reports


def first_divergence(reports: list) -> Optional[dict]:
    """The first record (in run order) whose replay differs, with its first differing field; skipped records (no
    function for their stage) never count."""
    for r in reports:
        if r["ok"] is False:
            where, what = r["diffs"][0]
            return {"file": r["file"], "stage": r["stage"], "rollout_id": r["rollout_id"], "step_id": r.get("step_id"),
                    "field": where, "difference": what}
    return None


def main(argv=None):
    import argparse

    ap = argparse.ArgumentParser(prog="relax_b200.utils.replay", description="Offline trajectory replay")
    sub = ap.add_subparsers(dest="cmd")
    for name in ("inspect", "validate", "replay"):
        sp = sub.add_parser(name)
        sp.add_argument("bundle")
        if name == "replay":
            sp.add_argument("--stage", default="all", help="reward, advantages, loss or all")
            sp.add_argument("--rollout", type=int, nargs="*", default=None)
            sp.add_argument("--atol", type=float, default=1e-6)
            sp.add_argument("--rtol", type=float, default=1e-5)
            sp.add_argument("--json", action="store_true", help="print the report as JSON")
    argv = list(argv) if argv is not None else None
    if argv and argv[0] not in ("inspect", "validate", "replay", "-h", "--help"):
        argv = ["replay"] + argv                       # the bare form: replay <bundle>
    a = ap.parse_args(argv)
    if a.cmd == "inspect":
        m = load_manifest(a.bundle)
        print(json.dumps({"identity": m.get("identity"), "ranks": m.get("ranks", [m.get("rank")]), "records": len(m["records"]),
                          "stages": sorted({r["stage"] for r in m["records"]}), "rollouts": sorted({r["rollout_id"] for r in m["records"]})},
                         indent=1))
        return 0
    if a.cmd == "validate":
        problems = validate_bundle(a.bundle)
        print("valid" if not problems else "\n".join(problems))
        return 0 if not problems else 1
    reps = replay_bundle(a.bundle, atol=a.atol, rtol=a.rtol, stages=None if a.stage == "all" else [a.stage], rollouts=a.rollout)
    first = first_divergence(reps)
    if a.json:
        print(json.dumps({"records": len(reps), "ok": sum(1 for r in reps if r["ok"]), "first_divergence": first}, indent=1))
    else:
        for r in reps:
            print(("OK   " if r["ok"] else "DIFF ") + r["file"] + "".join(f"\n      {w}: {d}" for w, d in r["diffs"]))
        if first:
            print(f"first divergence: rollout {first['rollout_id']} step {first['step_id']} stage {first['stage']} at {first['field']}: {first['difference']}")
    return 0 if all(r["ok"] for r in reps) else 1


if __name__ == "__main__":
    raise SystemExit(main())
