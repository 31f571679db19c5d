"""Radix tree over text prefixes that remembers, for every cached prefix, the exact token ids,
their sampling log-probs, the loss mask (1 on model-generated tokens) and the weight version that
produced them.  Multi-turn / agentic rollouts re-submit "conversation so far + new turn": the
cache returns the stored tokens of the longest known prefix, so a turn is neither re-tokenised
(tokenisation of a concatenation can differ from the concatenation of tokenisations) nor are its
log-probs recomputed.  Entries written by weights older than ``gc_threshold_k`` versions are
collected; least-recently-used leaves are evicted above ``max_tokens``.

Same contract as the reference middleware (relax/engine/router/middleware/radix_tree.py:100-620:
``find_longest_prefix``, ``insert``, ``remove``, ``gc_by_weight_version``, ``retrieve_from_text``).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional


class _Node:
    __slots__ = ("key", "tokens", "logp", "mask", "children", "parent", "last_access", "ref", "version")

    def __init__(self, key="", tokens=None, logp=None, mask=None, parent=None, version=None):
        self.key, self.tokens, self.logp, self.mask = key, tokens or [], logp or [], mask or []
        self.children: dict = {}      # edge text -> node (edges are never split: a split point need not be a token boundary)
        self.parent, self.version = parent, version
        self.last_access = time.monotonic()
        self.ref = 0


@dataclass
class Match:
    matched_prefix: str
    token_ids: List[int]
    logp: List[float]
    loss_mask: List[int]
    remaining: str
    node: object = field(repr=False, default=None)


class RadixCache:
    def __init__(self, tokenizer: Optional[Callable[[str], List[int]]] = None, max_tokens: int = 1 << 22,
                 gc_threshold_k: int = 5):
        self.root = _Node()
        self.tokenizer, self.max_tokens, self.gc_threshold_k = tokenizer, max_tokens, gc_threshold_k
        self.total_tokens = 0
        self._lock = threading.RLock()

    # ------------------------------------------------------------------ lookup
    def find_longest_prefix(self, text: str) -> Match:
        with self._lock:
            node, i = self.root, 0
            toks, lps, mask = [], [], []
            while i < len(text):
                child = None
                for key, c in node.children.items():   # longest edge that is a prefix of what is left
                    if text.startswith(key, i) and (child is None or len(key) > len(child.key)):
                        child = c
                if child is None:
                    break   # a partial match of an edge holds no token boundary: stop at the node above
                node, i = child, i + len(child.key)
                toks += node.tokens
                lps += node.logp
                mask += node.mask
                node.last_access = time.monotonic()
            return Match(text[:i], toks, lps, mask, text[i:], node)

    # ------------------------------------------------------------------ insert
    def insert(self, text: str, token_ids: List[int], logp: Optional[List[float]] = None,
               loss_mask: Optional[List[int]] = None, weight_version: Optional[int] = None) -> bool:
        """Store ``token_ids`` (and per-token ``logp`` / ``loss_mask``) for the whole of ``text``.  The part
        already cached is kept; only the new suffix (and its tokens beyond the cached ones) is added."""
        logp = list(logp) if logp is not None else [0.0] * len(token_ids)
        loss_mask = list(loss_mask) if loss_mask is not None else [0] * len(token_ids)
        if not (len(token_ids) == len(logp) == len(loss_mask)):
            raise ValueError("token_ids, logp and loss_mask must have one entry per token")
        with self._lock:
            m = self.find_longest_prefix(text)
            have = len(m.token_ids)
            if not m.remaining:
                self._touch_version(m.node, weight_version)
                return False
            if have > len(token_ids) or list(token_ids[:have]) != m.token_ids:
                raise ValueError("tokens of the cached prefix do not match the new sequence")
            node = m.node
            # the new suffix hangs off the deepest fully matched node; siblings may share leading characters
            child = _Node(m.remaining, list(token_ids[have:]), logp[have:], loss_mask[have:], node, weight_version)
            node.children[m.remaining] = child
            self._touch_version(node, weight_version)
            self.total_tokens += len(child.tokens)
            self._evict_if_needed(protect=child)
            return True

    def _touch_version(self, node, version):
        if version is None:
            return
        while node is not None and node is not self.root:
            if node.version is None or node.version < version:
                node.version = version
            node = node.parent

    # ------------------------------------------------------------------ removal / GC
    def _drop_subtree(self, node) -> int:
        n = len(node.tokens)
        for c in list(node.children.values()):
            n += self._drop_subtree(c)
        if node.parent is not None:
            node.parent.children.pop(node.key, None)
        self.total_tokens -= len(node.tokens)
        node.children = {}
        return n

    def remove(self, text: str) -> bool:
        with self._lock:
            m = self.find_longest_prefix(text)
            if m.remaining or m.node is self.root:
                return False
            self._drop_subtree(m.node)
            return True

    def gc_by_weight_version(self, current_version: int) -> int:
        """Drop every subtree whose entries were written more than ``gc_threshold_k`` weight versions ago."""
        limit = current_version - self.gc_threshold_k
        freed = 0
        with self._lock:
            stack = list(self.root.children.values())
            while stack:
                n = stack.pop()
                if n.version is not None and n.version < limit and n.ref == 0:
                    freed += self._drop_subtree(n)
                else:
                    stack.extend(n.children.values())
        return freed

    def _leaves(self):
        out, stack = [], list(self.root.children.values())
        while stack:
            n = stack.pop()
            if n.children:
                stack.extend(n.children.values())
            else:
                out.append(n)
        return out

    def _evict_if_needed(self, protect=None):
        while self.total_tokens > self.max_tokens:
            cands = [n for n in self._leaves() if n.ref == 0 and n is not protect]
            if not cands:
                return
            self._drop_subtree(min(cands, key=lambda n: n.last_access))

    # ------------------------------------------------------------------ convenience
    def retrieve_from_text(self, text: str, return_logprob: bool = True):
        """Tokens for ``text``: cached prefix + tokenizer on the rest (which is then cached with zero
        log-probs and loss mask 0 = not model-generated)."""
        m = self.find_longest_prefix(text)
        toks, lps, mask = list(m.token_ids), list(m.logp), list(m.loss_mask)
        if m.remaining:
            if self.tokenizer is None:
                raise ValueError("text extends beyond the cache and no tokenizer was given")
            extra = list(self.tokenizer(m.remaining))
            toks += extra
            lps += [0.0] * len(extra)
            mask += [0] * len(extra)
            self.insert(text, toks, lps, mask)
        return (toks, lps, mask) if return_logprob else (toks, mask)

    def stats(self) -> dict:
        with self._lock:
            n, stack = 0, [self.root]
            while stack:
                x = stack.pop()
                n += 1
                stack.extend(x.children.values())
            return {"nodes": n - 1, "tokens": self.total_tokens}

    def clear(self):
        with self._lock:
            self.root = _Node()
            self.total_tokens = 0
