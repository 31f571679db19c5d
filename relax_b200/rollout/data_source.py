"""Prompt sources for rollouts: a dataset cursor that hands out groups of
``n_samples_per_prompt`` pending samples and can be checkpointed, plus a
buffered variant that re-queues aborted (partial-rollout) samples first.

Counterpart of relax/engine/rollout/data_source.py (``RolloutDataSource``,
``RolloutDataSourceWithBuffer``: ``get_samples / add_samples / save / load``).
"""
from __future__ import annotations

import copy
import json
import os
import random
from typing import Callable, Optional, Sequence

import torch

from ..types import Sample


class SyntheticPromptDataset:
    """Random token prompts of fixed length (benchmarks / tests)."""

    def __init__(self, num_prompts: int, prompt_len: int, vocab_size: int, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.data = torch.randint(0, vocab_size, (num_prompts, prompt_len), generator=g)

    def __len__(self):
        return self.data.shape[0]

    def __getitem__(self, i):
        return {"prompt_tokens": self.data[i].tolist(), "label": None}


class JsonlPromptDataset:
    """``{"prompt": ..., "label": ...}`` per line; tokenised lazily by ``tokenize``."""

    def __init__(self, path: str, tokenize: Optional[Callable] = None, prompt_key="prompt", label_key="label",
                 metadata_key: str = "metadata"):
        """``path`` may list several files separated by commas.  Rows whose prompt ``tokenize`` rejects (returns
        None: longer than the prompt limit) are dropped at load time, so the epoch length is known up front."""
        self.rows = []
        for one in str(path).split(","):
            if one:
                with open(one, encoding="utf-8") as f:
                    self.rows += [json.loads(l) for l in f if l.strip()]
        self.tokenize, self.prompt_key, self.label_key, self.metadata_key = tokenize, prompt_key, label_key, metadata_key
        if tokenize is not None:
            kept = []
            for r in self.rows:
                toks = tokenize(r[prompt_key])
                if toks is not None:
                    r["_tokens"] = toks
                    kept.append(r)
            self.dropped = len(self.rows) - len(kept)
            self.rows = kept

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        r = self.rows[i]
        p = r[self.prompt_key]
        toks = r["_tokens"] if "_tokens" in r else list(p)
        return {"prompt": p, "prompt_tokens": toks, "label": r.get(self.label_key) if self.label_key else None,
                "metadata": r.get(self.metadata_key) or {}}


class RolloutDataSource:
    def __init__(self, dataset, n_samples_per_prompt: int, shuffle: bool = False, seed: int = 42):
        self.dataset, self.n = dataset, n_samples_per_prompt
        self.shuffle, self.seed = shuffle, seed
        self.epoch, self.offset = 0, 0
        self.sample_index, self.group_index = 0, 0
        self._order = self._make_order()

    def _make_order(self):
        idx = list(range(len(self.dataset)))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(idx)
        return idx

    def get_samples(self, num_groups: int) -> list[list[Sample]]:
        groups = []
        for _ in range(num_groups):
            if self.offset >= len(self._order):
                self.epoch += 1
                self.offset = 0
                self._order = self._make_order()
            row = self.dataset[self._order[self.offset]]
            self.offset += 1
            grp = []
            for _ in range(self.n):
                s = Sample(group_index=self.group_index, index=self.sample_index, prompt=row.get("prompt", ""),
                           tokens=list(row["prompt_tokens"]), label=row.get("label"),
                           metadata=dict(row.get("metadata") or {}))
                self.sample_index += 1
                grp.append(s)
            self.group_index += 1
            groups.append(grp)
        return groups

    def add_samples(self, groups):
        raise RuntimeError("this data source has no buffer; use RolloutDataSourceWithBuffer")

    def state_dict(self):
        return {"epoch": self.epoch, "offset": self.offset, "sample_index": self.sample_index,
                "group_index": self.group_index, "seed": self.seed}

    def load_state_dict(self, sd):
        self.epoch, self.offset = sd["epoch"], sd["offset"]
        self.sample_index, self.group_index = sd["sample_index"], sd["group_index"]
        self.seed = sd.get("seed", self.seed)
        self._order = self._make_order()

    def save(self, directory: str, rollout_id: int):
        os.makedirs(os.path.join(directory, "dataset"), exist_ok=True)
        torch.save(self.state_dict(), os.path.join(directory, "dataset", f"global_dataset_state_dict_{rollout_id}.pt"))

    def load(self, directory: str, rollout_id: int) -> bool:
        p = os.path.join(directory, "dataset", f"global_dataset_state_dict_{rollout_id}.pt")
        if not os.path.exists(p):
            return False
        self.load_state_dict(torch.load(p))
        return True


class RolloutDataSourceWithBuffer(RolloutDataSource):
    """Aborted groups go to a buffer and are served before fresh prompts."""

    def __init__(self, *a, buffer_filter: Optional[Callable] = None, **k):
        super().__init__(*a, **k)
        self.buffer: list = []
        self.buffer_filter = buffer_filter or (lambda buf, n: [buf.pop(0) for _ in range(min(n, len(buf)))])

    def get_samples(self, num_groups: int):
        out = self.buffer_filter(self.buffer, num_groups)
        if len(out) < num_groups:
            out += super().get_samples(num_groups - len(out))
        return out

    def add_samples(self, groups):
        for g in groups:
            if len(g) != self.n:
                raise ValueError(f"group of {len(g)} samples, expected {self.n}")
            self.buffer.append(g)

    def state_dict(self):
        sd = super().state_dict()
        sd["buffer"] = [[s.to_dict() for s in g] for g in self.buffer]
        return sd

    def load_state_dict(self, sd):
        super().load_state_dict(sd)
        self.buffer = [[Sample.from_dict(d) for d in g] for g in sd.get("buffer", [])]
