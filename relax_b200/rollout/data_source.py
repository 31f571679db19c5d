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


class SyntheticImagePromptDataset:
    """Random prompts with one random "image" each: ``text_len`` tokens, a run of image placeholders, ``text_len``
    tokens.  Patches are Gaussian noise of the tower's patch size (benchmarks / tests of the vision-language loop).
    Rows are made on access from a per-row seed, so a large ``num_prompts`` costs nothing up front (one 448 x 448 image
    is 4.8 MB of patches)."""

    def __init__(self, num_prompts: int, text_len: int, vocab_size: int, image_token_id: int, grid_hw=(8, 8),
                 patch_dim: int = 1176, merge: int = 2, seed: int = 0):
        gh, gw = grid_hw
        assert gh % merge == 0 and gw % merge == 0
        self.n, self.text_len, self.vocab, self.img_id = num_prompts, text_len, vocab_size, image_token_id
        self.gh, self.gw, self.patch_dim, self.merge, self.seed = gh, gw, patch_dim, merge, seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        if not 0 <= i < self.n:
            raise IndexError(i)
        g = torch.Generator().manual_seed(self.seed * 1000003 + i)
        n_img = self.gh * self.gw // (self.merge * self.merge)
        text = torch.randint(0, self.vocab, (2 * self.text_len,), generator=g)
        text[text == self.img_id] = (self.img_id + 1) % self.vocab
        toks = text[:self.text_len].tolist() + [self.img_id] * n_img + text[self.text_len:].tolist()
        return {"prompt_tokens": toks, "label": None,
                "multimodal": {"pixel_patches": torch.randn(self.gh * self.gw, self.patch_dim, generator=g),
                               "grid_thw": torch.tensor([[1, self.gh, self.gw]])}}


class JsonlPromptDataset:
    """``{"prompt": ..., "label": ...}`` per line; tokenised lazily by ``tokenize``."""

    def __init__(self, path: str, tokenize: Optional[Callable] = None, prompt_key="prompt", label_key="label",
                 metadata_key: str = "metadata", tool_key: Optional[str] = None, image_key: Optional[str] = None,
                 image_token_id: Optional[int] = None, multimodal_config=None):
        """``path`` may list several files separated by commas.  Rows whose prompt ``tokenize`` rejects (returns
        None: longer than the prompt limit) are dropped at load time, so the epoch length is known up front."""
        self.rows = []
        for one in str(path).split(","):
            if one:
                with open(one, encoding="utf-8") as f:
                    self.rows += [json.loads(l) for l in f if l.strip()]
        self.tokenize, self.prompt_key, self.label_key, self.metadata_key = tokenize, prompt_key, label_key, metadata_key
        # rows with images (``image_key``: a path / data URI or a list of them): the prompt carries ONE placeholder
        # token per image, expanded to the image's token count when the row is read; the patches ride along
        self.image_key, self.image_token_id, self.mm_cfg = image_key, image_token_id, multimodal_config
        if image_key is not None and image_token_id is None:
            raise ValueError("image_key needs image_token_id (the id of the placeholder the prompt contains)")
        if tokenize is not None:
            kept = []
            for r in self.rows:
                tools = r.get(tool_key) if tool_key else None
                if isinstance(tools, str):
                    tools = json.loads(tools) if tools.strip() else None
                toks = tokenize(r[prompt_key], tools=tools) if tools else tokenize(r[prompt_key])
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
        out = {"prompt": p, "prompt_tokens": toks, "label": r.get(self.label_key) if self.label_key else None,
               "metadata": r.get(self.metadata_key) or {}}
        imgs = r.get(self.image_key) if self.image_key else None
        if imgs:
            from ..data.multimodal import expand_placeholders, process_multimodal_info

            imgs = [imgs] if isinstance(imgs, (str, bytes)) else list(imgs)
            mm = process_multimodal_info([{"role": "user", "content": [{"type": "image", "image": x} for x in imgs]}], self.mm_cfg)
            out["prompt_tokens"] = expand_placeholders(toks, self.image_token_id, mm["num_tokens"]["image"])
            out["multimodal"] = {"pixel_patches": mm["pixel_values"], "grid_thw": mm["image_grid_thw"]}
        return out


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
                           metadata=dict(row.get("metadata") or {}), multimodal_train_inputs=row.get("multimodal"))
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


class _NoPrompts:
    """Stand-in dataset of a data source without a global dataset: every row is an empty prompt."""

    def __len__(self):
        return 1 << 62

    def __getitem__(self, i):
        return {"prompt": "", "prompt_tokens": [], "label": None, "metadata": {}}


class ShellDataSource(RolloutDataSource):
    """``--disable-rollout-global-dataset``: no prompt dataset is loaded; the source hands out numbered, empty samples
    and the rollout function brings its own data (relax/engine/rollout/data_source.py:169-231 - ``dataset`` stays
    None, groups of ``Sample()`` shells; nothing is saved or loaded for it)."""

    def __init__(self, n_samples_per_prompt: int):
        super().__init__(_NoPrompts(), n_samples_per_prompt, shuffle=False)

    def _make_order(self):
        return range(len(self.dataset))

    def save(self, directory: str, rollout_id: int):
        pass


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

    def get_buffered(self, num_groups: int) -> list:
        """Up to ``num_groups`` groups from the buffer only (the buffer is local to an engine replica)."""
        return self.buffer_filter(self.buffer, num_groups)

    def get_fresh(self, num_groups: int) -> list:
        """Fresh prompt groups from the dataset, bypassing the buffer (the global stream every replica slices)."""
        return super().get_samples(num_groups)

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


class StreamingRolloutDataSource:
    """Prompts read lazily from (possibly huge) JSONL files through a shuffle buffer, epoch after epoch
    (``--use-streaming-dataset``, ``--streaming-buffer-size``; relax/utils/data/streaming_dataset.py).  Memory holds
    ``buffer_size`` rows, not the data set.  The order is a pure function of ``(seed, epoch)``, so a resumed run
    replays the stream up to the saved position and continues with exactly the prompts the original run would
    have drawn."""

    def __init__(self, paths, tokenize: Optional[Callable], n_samples_per_prompt: int, buffer_size: int = 1024, seed: int = 42,
                 prompt_key: str = "prompt", label_key: Optional[str] = "label", metadata_key: str = "metadata", shuffle: bool = True):
        self.paths = [p for p in (paths.split(",") if isinstance(paths, str) else list(paths)) if p]
        self.tokenize, self.n = tokenize, n_samples_per_prompt
        self.buffer_size, self.seed, self.shuffle = max(1, buffer_size), seed, shuffle
        self.prompt_key, self.label_key, self.metadata_key = prompt_key, label_key, metadata_key
        self.epoch, self.consumed = 0, 0           # rows handed out in the current epoch
        self.sample_index, self.group_index = 0, 0
        self._it = self._rows(self.epoch)

    def _raw(self):
        for p in self.paths:
            with open(p, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        yield json.loads(line)

    def _rows(self, epoch: int):
        rng = random.Random(self.seed * 1000003 + epoch)
        buf = []
        for r in self._raw():
            toks = self.tokenize(r[self.prompt_key]) if self.tokenize else list(r[self.prompt_key])
            if toks is None:
                continue
            item = {"prompt": r[self.prompt_key], "prompt_tokens": toks, "label": r.get(self.label_key) if self.label_key else None,
                    "metadata": r.get(self.metadata_key) or {}}
            if not self.shuffle:
                yield item
                continue
            buf.append(item)
            if len(buf) >= self.buffer_size:
                yield buf.pop(rng.randrange(len(buf)))
        rng.shuffle(buf)
        yield from buf

    def _next_row(self):
        for _ in range(2):
            try:
                row = next(self._it)
                self.consumed += 1
                return row
            except StopIteration:
                if self.consumed == 0:
                    raise ValueError(f"no usable prompt in {self.paths}")
                self.epoch, self.consumed = self.epoch + 1, 0
                self._it = self._rows(self.epoch)
        raise RuntimeError("unreachable")

    def get_samples(self, num_groups: int) -> list:
        groups = []
        for _ in range(num_groups):
            row = self._next_row()
            grp = []
            for _ in range(self.n):
                grp.append(Sample(group_index=self.group_index, index=self.sample_index, prompt=row["prompt"],
                                  tokens=list(row["prompt_tokens"]), label=row["label"], metadata=dict(row["metadata"])))
                self.sample_index += 1
            self.group_index += 1
            groups.append(grp)
        return groups

    def add_samples(self, groups):
        raise RuntimeError("the streaming source has no buffer for returned samples")

    def state_dict(self):
        return {"epoch": self.epoch, "consumed": self.consumed, "sample_index": self.sample_index,
                "group_index": self.group_index, "seed": self.seed}

    def load_state_dict(self, sd):
        self.seed = sd.get("seed", self.seed)
        self.epoch, self.sample_index, self.group_index = sd["epoch"], sd["sample_index"], sd["group_index"]
        self._it = self._rows(self.epoch)
        self.consumed = 0
        for _ in range(sd["consumed"]):       # replay to the saved position
            next(self._it)
            self.consumed += 1
