"""Speculative decoding in the rollout engine, drafted by the model's own multi-token-prediction (MTP) block.

What the reference gets from its serving engine with ``--sglang-speculative-algorithm EAGLE/NEXTN`` on MTP-trained
models (the engine side is outside the reference's tree; docs/en/guide/mtp-rl-training.md describes the pairing with
``--enable-mtp-training``): every scheduler iteration proposes one more token per request with the cheap MTP block and
checks it with the policy in the same pass that produces the next token anyway, so an accepted proposal yields two
tokens for one pass over the weights - and decode is bound by reading the weights.

One iteration for a request whose newest token ``x_t`` has not been fed yet and whose proposal for the next one is ``d``:

1. *Verify*: the policy runs on two rows, ``x_t`` at position ``t`` and ``d`` at position ``t + 1``
   (:meth:`RolloutWeights.forward_rows`; both rows write their K/V first, the second row attends to the first).
2. *Sample*: ``y1`` from the first row's distribution with the request's own sampling parameters, exactly as without
   speculation.  If ``y1 == d`` the second row was computed on the right prefix and ``y2`` is sampled from it.
   The proposal is a point mass (the block's arg-max), so "keep what the policy sampled" IS the speculative-sampling
   rule: the proposal is accepted with probability ``p(d)`` and the output is distributed as ``p`` either way.  The
   recorded log-probs are the policy's - the trainer sees an on-policy sample.
3. *Draft*: the MTP block runs on the accepted positions (its input at position ``i`` is the policy's pre-norm hidden
   state of ``i`` and the embedding of token ``i + 1``) and its arg-max at the last one is the next proposal.  The
   block keeps its own K/V cache as layer ``num_layers`` of the paged cache, under the same block tables.

With ``speculative_steps = K > 1`` the block is chained: after the draft pass on true hidden states, ``K - 1`` more
single-row passes feed the block its OWN output hidden and its last proposal (the way EAGLE-style drafters run a one-
layer head for several steps), the verify pass carries ``K + 1`` rows per request, and proposals are accepted from the
left until the policy's sample differs.  The block's cache rows written from its own hidden are provisional: the next
draft pass rewrites the accepted positions from the policy's hidden states.

A rejected proposal leaves a stale K/V row behind the accepted tokens; it lies beyond the context length of every later
read until the next iteration overwrites it.  After a prefill the block is run over the whole prompt once (followers of a shared
prompt copy the leader's cache and only redo the last position, which depends on their own first token).

The step is host-driven (no windowed CUDA graph): the number of rows per request changes from step to step.
"""
from __future__ import annotations

import torch

from .. import ops


class SpeculativeMixin:
    """Methods of :class:`~relax_b200.rollout.engine.RolloutEngine` used when ``speculative`` is on."""

    def _grow(self, r, p: int):
        """Blocks of ``r`` cover position ``p``."""
        bs = self.block_size
        while p // bs >= len(r.blocks):
            r.blocks.append(self.bm.alloc())
            r._reserve = max(0, r._reserve - 1)

    def _room(self, r) -> int:
        """How many proposals the next verify pass of ``r`` may carry: every accepted proposal is one more token, and
        one token comes from the pass anyway."""
        return max(0, min(self.speculative_steps, r.params.max_new_tokens - len(r.output) - 1,
                          self._max_model_len() - r.num_tokens - 1))

    def _chain(self, reqs, first_logits, h_out):
        """Proposals of ``reqs`` from the draft pass on true hidden states (``first_logits`` / ``h_out``: one row per
        request, the block's logits and output hidden at the request's last accepted position), extended to
        ``speculative_steps`` by running the block on its own output."""
        v = self.cfg.vocab_size
        bs = self.block_size
        d = first_logits[:, :v].argmax(-1)
        drafts = [[x] for x in d.tolist()]
        live = [j for j, r in enumerate(reqs) if self._room(r) > 1]
        step = 1
        while live:
            rows = torch.tensor(live, device=h_out.device)
            pos, ctx, slots, bt = [], [], [], []
            for j in live:
                r = reqs[j]
                p = r.num_tokens - 2 + step           # the position whose (stand-in) hidden state feeds this pass
                self._grow(r, p)
                pos.append(p + r.pos_delta)
                ctx.append(p + 1)
                slots.append(r.blocks[p // bs] * bs + p % bs)
            maxb = (max(len(reqs[j].blocks) for j in live) + 7) // 8 * 8
            bt = [reqs[j].blocks + [0] * (maxb - len(reqs[j].blocks)) for j in live]
            p_t, c_t, s_t, b_t = self._stage([(pos, torch.int64), (ctx, torch.int32), (slots, torch.int64), (bt, torch.int32)])
            logits, h_new = self.weights.forward_mtp_rows(h_out.index_select(0, rows), d.index_select(0, rows), p_t, b_t, c_t, s_t,
                                                          self.kv, self.tp, return_hidden=True)
            nxt = logits[:, :v].argmax(-1)
            h_out = h_out.clone()
            h_out[rows] = h_new.to(h_out.dtype)
            d = d.clone()
            d[rows] = nxt
            for j, x in zip(live, nxt.tolist()):
                drafts[j].append(x)
            step += 1
            live = [j for j in live if self._room(reqs[j]) > step]
        for r, dr in zip(reqs, drafts):
            r._draft = dr

    # ------------------------------------------------------------------ after a prefill
    def _draft_after_prefill(self, reqs, leaders, h_all, cu, slots_t, pos_t, cu_t, row_of):
        """Fill the MTP block's cache for the prompts and set every request's first proposals."""
        L = self.cfg.num_layers
        bs = self.block_size
        if leaders:
            nxt = []
            for r in leaders:
                ctx = r.prompt + r.output            # the prompt and the token sampled just now
                nxt += ctx[1:]
            (nxt_t,) = self._stage([(nxt, torch.int64)])
            last = torch.tensor([b - 1 for b in cu[1:]], device=self.device)
            logits, ho = self.weights.forward_mtp_prefill(h_all, nxt_t, pos_t, cu_t, slots_t, self.kv, last, self.tp,
                                                          max_seqlen=max(b - a for a, b in zip(cu, cu[1:])))
            alive = [j for j, r in enumerate(leaders) if r.status != "finished"]
            if alive:
                sel = torch.tensor(alive, device=logits.device)
                self._chain([leaders[j] for j in alive], logits.index_select(0, sel), ho.index_select(0, sel))
        followers = [r for r in reqs if r._lead is not None and r.status != "finished"]
        if followers:
            rows_h, toks, pos, ctx, slots, bt = [], [], [], [], [], []
            maxb = (max(len(r.blocks) for r in followers) + 7) // 8 * 8
            for r in followers:
                lead = r._lead
                n = len(r.prompt)
                for j in range((n - 1) // bs, len(lead.blocks)):       # the leader's tail blocks of the block's own cache
                    if j < len(r.blocks):
                        self.kv[L, :, r.blocks[j]] = self.kv[L, :, lead.blocks[j]]
                rows_h.append(cu[row_of[id(lead)] + 1] - 1)
                toks.append(r.output[-1])
                pos.append(n - 1 + r.pos_delta)
                ctx.append(n)
                slots.append(r.blocks[(n - 1) // bs] * bs + (n - 1) % bs)
                bt.append(r.blocks + [0] * (maxb - len(r.blocks)))
            rows_t, tok_t, p_t, c_t, s_t, bt_t = self._stage([(rows_h, torch.int64), (toks, torch.int64), (pos, torch.int64),
                                                               (ctx, torch.int32), (slots, torch.int64), (bt, torch.int32)])
            logits, ho = self.weights.forward_mtp_rows(h_all.index_select(0, rows_t), tok_t, p_t, bt_t, c_t, s_t, self.kv, self.tp,
                                                       return_hidden=True)
            self._chain(followers, logits, ho)

    # ------------------------------------------------------------------ one decode iteration
    def _decode_speculative(self):
        reqs = self.running
        bs = self.block_size
        v = self.cfg.vocab_size
        # rows: the newest token of every request, then as many of its proposals as it may still take
        owner, first_row, n_draft = [], [], []
        tok, pos, ctx, slots = [], [], [], []
        for i, r in enumerate(reqs):
            t = r.num_tokens - 1
            dr = list(getattr(r, "_draft", None) or [])[: self._room(r)]
            n_draft.append(len(dr))
            first_row.append(len(tok))
            for j, x in enumerate([r.output[-1] if r.output else r.prompt[-1]] + dr):
                p = t + j
                self._grow(r, p)
                owner.append(i)
                tok.append(x)
                pos.append(p + r.pos_delta)
                ctx.append(p + 1)
                slots.append(r.blocks[p // bs] * bs + p % bs)
            r._draft = dr
        maxb = (max(len(r.blocks) for r in reqs) + 7) // 8 * 8
        bt = [reqs[i].blocks + [0] * (maxb - len(reqs[i].blocks)) for i in owner]
        tok_t, pos_t, ctx_t, slots_t, bt_t = self._stage([(tok, torch.int64), (pos, torch.int64), (ctx, torch.int32),
                                                           (slots, torch.int64), (bt, torch.int32)])
        logits, h = self.weights.forward_rows(tok_t, pos_t, bt_t, ctx_t, slots_t, self.kv, self.tp)
        R = len(tok)
        self.stats["decode_tokens"] += R
        # one sampling call for all rows; row j + 1 of a request counts only if proposals 1 .. j + 1 were all accepted
        u = torch.rand(R, generator=self.gen)
        temp, topk, topp, u = self._stage([([reqs[i].params.temperature for i in owner], torch.float32),
                                           ([reqs[i].params.top_k for i in owner], torch.int64),
                                           ([reqs[i].params.top_p for i in owner], torch.float32),
                                           (u.tolist(), torch.float32)])
        y, lp = ops.sample(logits[:, :v], temp, topk, topp, u)
        y_l, lp_l = y.tolist(), lp.tolist()
        self.stats["d2h_bytes"] = self.stats.get("d2h_bytes", 0) + R * 12
        # accepted positions per request -> rows of the draft pass
        m_rows, m_tok, m_pos, m_ctx, m_slots, m_owner, last_of = [], [], [], [], [], [], {}
        for i, r in enumerate(reqs):
            a = first_row[i]
            self._append_tokens([r], [y_l[a]], [lp_l[a]])
            took = 1
            self.stats["spec_draft_tokens"] = self.stats.get("spec_draft_tokens", 0) + n_draft[i]
            r.spec_draft += n_draft[i]
            for j in range(n_draft[i]):
                if y_l[a + j] != r._draft[j] or r.status == "finished":
                    break
                self._append_tokens([r], [y_l[a + j + 1]], [lp_l[a + j + 1]])
                self.stats["spec_accepted_tokens"] = self.stats.get("spec_accepted_tokens", 0) + 1
                r.spec_accept += 1
                took += 1
            r.spec_verify += 1
            r._draft = None
            if r.status == "finished":
                continue
            n = r.num_tokens                      # tokens x_0 .. x_{n-1}; the block is due at positions n-1-took .. n-2
            for j in range(took):
                p = n - 1 - took + j
                m_rows.append(a + j)              # the trunk's hidden state of position p is row a + j of this pass
                m_tok.append(r.output[len(r.output) - took + j])      # the token that follows position p
                m_pos.append(p + r.pos_delta)
                m_ctx.append(p + 1)
                m_slots.append(r.blocks[p // bs] * bs + p % bs)
                m_owner.append(i)
            last_of[i] = len(m_rows) - 1
        self.stats["spec_verify_steps"] = self.stats.get("spec_verify_steps", 0) + 1
        if not m_rows:
            return
        m_bt = [reqs[i].blocks + [0] * (maxb - len(reqs[i].blocks)) for i in m_owner]
        alive = sorted(last_of)
        out_rows = [last_of[i] for i in alive]
        rows_t, t_t, p_t, c_t, s_t, b_t, o_t = self._stage([(m_rows, torch.int64), (m_tok, torch.int64), (m_pos, torch.int64),
                                                            (m_ctx, torch.int32), (m_slots, torch.int64), (m_bt, torch.int32),
                                                            (out_rows, torch.int64)])
        dl, ho = self.weights.forward_mtp_rows(h.index_select(0, rows_t), t_t, p_t, b_t, c_t, s_t, self.kv, self.tp, out_rows=o_t,
                                               return_hidden=True)
        self._chain([reqs[i] for i in alive], dl, ho)
