"""Supervised fine-tuning data: chat-template rendering with a loss mask on the assistant turns,
a streaming reader over JSONL shards, and greedy packing into token-budgeted batches.

Mirrors what the reference's streaming SFT dataset produces (relax/engine/sft/dataset/streaming.py:
messages -> token ids + loss mask, sharded by data-parallel rank, resumable by (file, line) cursor)
without its tokenizer-processor pool; tokenisation is a callable so tests use a toy tokenizer.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable, Iterable, Iterator, List, Optional, Sequence


def render_chat(messages: Sequence[dict], tokenize: Callable[[str], List[int]], bos: Optional[int] = None,
                eos: Optional[int] = None, role_prefix: Callable[[str], str] = lambda r: f"<|{r}|>\n",
                turn_suffix: str = "\n") -> tuple:
    """Token ids and loss mask (1 on assistant content and its end marker) of a conversation."""
    toks: List[int] = [] if bos is None else [bos]
    mask: List[int] = [0] * len(toks)
    for m in messages:
        head = tokenize(role_prefix(m["role"]))
        body = tokenize(m["content"] + turn_suffix)
        toks += head
        mask += [0] * len(head)
        train = 1 if m["role"] == "assistant" else 0
        toks += body
        mask += [train] * len(body)
        if train and eos is not None:
            toks.append(eos)
            mask.append(1)
    return toks, mask


def to_train_sample(tokens: List[int], mask: List[int], max_len: Optional[int] = None) -> Optional[dict]:
    """The trainer's convention: ``response_lengths`` = length of the suffix starting at the first trained
    token; ``loss_masks`` covers that suffix.  Returns None when nothing is trained."""
    if max_len is not None:
        tokens, mask = tokens[:max_len], mask[:max_len]
    if 1 not in mask:
        return None
    first = mask.index(1)
    first = max(first, 1)   # position 0 has no context to be predicted from
    return {"tokens": tokens, "response_length": len(tokens) - first, "loss_mask": mask[first:]}


@dataclass
class SFTCursor:
    file_index: int = 0
    line: int = 0
    epoch: int = 0


class StreamingSFTDataset:
    """Iterates samples from JSONL files (``{"messages": [...]}`` or ``{"prompt":..., "response":...}``), keeping
    every ``dp_size``-th sample for this rank; ``state_dict``/``load_state_dict`` resume mid-file."""

    def __init__(self, files: Sequence[str], tokenize: Callable[[str], List[int]], dp_rank: int = 0, dp_size: int = 1,
                 max_len: Optional[int] = None, eos: Optional[int] = None, epochs: Optional[int] = 1):
        self.files, self.tokenize = list(files), tokenize
        self.dp_rank, self.dp_size, self.max_len, self.eos, self.epochs = dp_rank, dp_size, max_len, eos, epochs
        self.cursor = SFTCursor()
        self._count = 0

    def state_dict(self) -> dict:
        return {"file_index": self.cursor.file_index, "line": self.cursor.line, "epoch": self.cursor.epoch,
                "count": self._count}

    def load_state_dict(self, st: dict):
        self.cursor = SFTCursor(st["file_index"], st["line"], st["epoch"])
        self._count = st.get("count", 0)

    def _parse(self, rec: dict) -> Optional[dict]:
        if "messages" in rec:
            msgs = rec["messages"]
        else:
            msgs = [{"role": "user", "content": rec["prompt"]}, {"role": "assistant", "content": rec["response"]}]
        toks, mask = render_chat(msgs, self.tokenize, eos=self.eos)
        return to_train_sample(toks, mask, self.max_len)

    def __iter__(self) -> Iterator[dict]:
        while self.epochs is None or self.cursor.epoch < self.epochs:
            while self.cursor.file_index < len(self.files):
                with open(self.files[self.cursor.file_index]) as f:
                    for ln, line in enumerate(f):
                        if ln < self.cursor.line:
                            continue
                        self.cursor.line = ln + 1
                        if not line.strip():
                            continue
                        mine = self._count % self.dp_size == self.dp_rank
                        self._count += 1
                        if not mine:
                            continue
                        s = self._parse(json.loads(line))
                        if s is not None:
                            yield s
                self.cursor.file_index += 1
                self.cursor.line = 0
            self.cursor = SFTCursor(0, 0, self.cursor.epoch + 1)


def pack_batches(samples: Iterable[dict], max_tokens: int, max_samples: Optional[int] = None) -> Iterator[dict]:
    """Group consecutive samples into trainer batches of at most ``max_tokens`` tokens."""
    cur: List[dict] = []
    n = 0
    for s in samples:
        L = len(s["tokens"])
        if cur and (n + L > max_tokens or (max_samples and len(cur) >= max_samples)):
            yield as_batch(cur)
            cur, n = [], 0
        cur.append(s)
        n += L
    if cur:
        yield as_batch(cur)


def as_batch(samples: Sequence[dict]) -> dict:
    return {"tokens": [s["tokens"] for s in samples],
            "response_lengths": [s["response_length"] for s in samples],
            "loss_masks": [s["loss_mask"] for s in samples]}


def batches_with_cursor(ds: StreamingSFTDataset, samples_per_batch: int) -> Iterator[tuple]:
    """``(batch, dataset state after its last sample)`` pairs: a run that stores the state of the last batch it TRAINED
    on resumes with the next unseen sample, however far a prefetcher had read ahead."""
    cur: List[dict] = []
    for s in ds:
        cur.append(s)
        if len(cur) >= samples_per_batch:
            yield as_batch(cur), ds.state_dict()
            cur = []
    if cur:
        yield as_batch(cur), ds.state_dict()


class Prefetcher:
    """A background thread that keeps up to ``depth`` items of an iterator ready (the tokenisation of the next SFT
    batches overlaps the training step; relax/engine/sft/dataset/streaming.py prefetch buffer,
    ``--sft-prefetch-buffer-size``).  Exceptions of the producer surface at the consumer."""

    _END = object()

    def __init__(self, it: Iterable, depth: int = 4):
        import queue
        import threading

        self._q: "queue.Queue" = queue.Queue(maxsize=max(1, int(depth)))
        self._stop = threading.Event()

        def run():
            try:
                for x in it:
                    while not self._stop.is_set():
                        try:
                            self._q.put(x, timeout=0.1)
                            break
                        except queue.Full:
                            continue
                    if self._stop.is_set():
                        return
                self._q.put(self._END)
            except BaseException as e:  # noqa: BLE001 - handed to the consumer
                self._q.put(e)

        self._t = threading.Thread(target=run, daemon=True, name="sft-prefetch")
        self._t.start()

    def __iter__(self):
        return self

    def __next__(self):
        x = self._q.get()
        if x is self._END:
            raise StopIteration
        if isinstance(x, BaseException):
            raise x
        return x

    def close(self):
        self._stop.set()
