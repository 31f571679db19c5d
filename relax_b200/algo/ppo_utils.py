"""RL math on packed token streams.

Every function here works on *packed* 1-D tensors (all response tokens of a
micro-batch concatenated) plus a segment description, so one launch covers the
whole micro-batch instead of one Python iteration per sample.  List-of-tensor
convenience wrappers are provided for callers that hold per-sample tensors.

Behavioural parity targets (reference paths inside its project):
  relax/utils/training/ppo_utils.py:100-139   KL estimators k1/k2/k3/low_var_kl
  relax/utils/training/ppo_utils.py:142-209   OPSM mask, GSPO sequence KL
  relax/utils/training/ppo_utils.py:212-461   SAPO / CISPO / RLOO / PPO-clip / M2PO
  relax/utils/training/ppo_utils.py:654-1189  GRPO returns, RLOO, REINFORCE++, GAE
  relax/utils/utils.py:180-240                group reward normalisation
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

import torch

class _PinnedRing:
    """A few pinned staging buffers reused round-robin.  ``tensor.pin_memory()`` per call would ask the driver for a new
    pinned block for every new size (a slow call that also stalls the device); here a slot grows in powers of two and is
    reused once the copy that last read it has run (an event per slot; with 8 slots the wait is never taken in practice)."""

    SLOTS = 8

    def __init__(self):
        import threading

        self.bufs = [None] * self.SLOTS
        self.events = [None] * self.SLOTS
        self.i = 0
        self.lock = threading.Lock()       # role threads of one process (actor, forward roles) stage concurrently

    def stage(self, t: torch.Tensor, device: torch.device) -> torch.Tensor:
        with self.lock:
            return self._stage(t, device)

    def _stage(self, t: torch.Tensor, device: torch.device) -> torch.Tensor:
        nbytes = t.numel() * t.element_size()
        k = self.i
        self.i = (self.i + 1) % self.SLOTS
        if self.events[k] is not None:
            self.events[k].synchronize()
        if self.bufs[k] is None or self.bufs[k].numel() < nbytes:
            self.bufs[k] = torch.empty(max(4096, 1 << max(0, (nbytes - 1).bit_length())), dtype=torch.uint8, pin_memory=True)
        src = self.bufs[k][:nbytes].view(t.dtype).view(t.shape)
        src.copy_(t)
        out = src.to(device, non_blocking=True)
        ev = self.events[k] or torch.cuda.Event()
        ev.record(torch.cuda.current_stream(device))
        self.events[k] = ev
        return out


_RING = None


def to_device_async(t: torch.Tensor, device) -> torch.Tensor:
    """Host tensor -> ``device`` without blocking the host: through a pinned staging buffer with a non-blocking copy.
    A plain ``.to(device)`` from pageable memory waits for everything queued on the stream, which stops the host from
    running ahead of the GPU."""
    global _RING
    if device is None:
        return t
    device = torch.device(device)
    if device.type != "cuda" or t.is_cuda or t.numel() == 0:
        return t.to(device)
    if _RING is None:
        _RING = _PinnedRing()
    return _RING.stage(t.contiguous(), device)


# --------------------------------------------------------------------------- segments


@dataclass
class Segments:
    """Describes how a packed 1-D tensor splits into per-sample pieces."""

    lengths: torch.Tensor  # [B] int64 (on the data device)
    # the same lengths on the host when the caller had them there: ``split`` / ``ids`` then need no device read (a
    # ``tolist()`` or a ``repeat_interleave`` without a known output size blocks the host until the stream drains)
    host: "list | None" = None

    @staticmethod
    def from_lengths(lengths: Sequence[int] | torch.Tensor, device=None) -> "Segments":
        if torch.is_tensor(lengths):
            return Segments(lengths.to(device=device, dtype=torch.int64))
        host = [int(x) for x in lengths]
        return Segments(to_device_async(torch.tensor(host, dtype=torch.int64), device), host)

    @property
    def num(self) -> int:
        return int(self.lengths.numel())

    @property
    def cu(self) -> torch.Tensor:
        z = torch.zeros(1, dtype=torch.int64, device=self.lengths.device)
        return torch.cat([z, torch.cumsum(self.lengths, 0)])

    @property
    def ids(self) -> torch.Tensor:
        total = sum(self.host) if self.host is not None else None
        return torch.repeat_interleave(torch.arange(self.num, device=self.lengths.device), self.lengths, output_size=total)

    def seg_sum(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.zeros(self.num, dtype=x.dtype, device=x.device)
        return out.index_add(0, self.ids.to(x.device), x)

    def expand(self, per_seg: torch.Tensor) -> torch.Tensor:
        return per_seg[self.ids.to(per_seg.device)]

    def split(self, x: torch.Tensor) -> list[torch.Tensor]:
        return list(torch.split(x, self.host if self.host is not None else self.lengths.tolist()))


def pack(xs: Sequence[torch.Tensor]) -> tuple[torch.Tensor, Segments]:
    seg = Segments.from_lengths([int(x.numel()) for x in xs], device=xs[0].device if xs else None)
    return (torch.cat(list(xs)) if xs else torch.zeros(0)), seg


# --------------------------------------------------------------------------- KL estimators


def compute_approx_kl(log_probs, log_probs_base, kl_loss_type: str = "k1", importance_ratio=None):
    """Schulman's k1/k2/k3 estimators of KL(pi || base) from samples of pi.

    ``low_var_kl`` is k3 clamped to [-10, 10].  An optional importance ratio
    (pi_theta / pi_old) multiplies the estimate before the clamp.
    """
    d = log_probs.float() - log_probs_base.float()
    if kl_loss_type == "k1":
        kl = d
    elif kl_loss_type == "k2":
        kl = 0.5 * d * d
    elif kl_loss_type in ("k3", "low_var_kl"):
        nd = -d
        kl = torch.exp(nd) - 1.0 - nd
    else:
        raise ValueError(f"Unknown kl_loss_type: {kl_loss_type}")
    if importance_ratio is not None:
        kl = importance_ratio * kl
    if kl_loss_type == "low_var_kl":
        kl = kl.clamp(-10.0, 10.0)
    return kl


# --------------------------------------------------------------------------- sequence-level helpers


def masked_seq_mean(x: torch.Tensor, mask: torch.Tensor, seg: Segments) -> torch.Tensor:
    """Per-sample masked mean, denominator clamped to >= 1."""
    num = seg.seg_sum(x * mask)
    den = seg.seg_sum(mask.to(x.dtype)).clamp_min(1)
    return num / den


def compute_gspo_kl(log_probs, old_log_probs, loss_mask, seg: Segments, expand_seg: Segments | None = None):
    """Sequence-level ``old - new`` masked mean broadcast back over tokens.

    ``seg`` describes the tensors the mean is taken over (full responses);
    ``expand_seg`` the shape to broadcast to (the context-parallel local slice);
    it defaults to ``seg``.
    """
    seq_kl = masked_seq_mean(old_log_probs - log_probs, loss_mask, seg)
    return (expand_seg or seg).expand(seq_kl)


def compute_opsm_mask(log_probs, old_log_probs, advantages, loss_mask, seg: Segments, opsm_delta: float):
    """Off-policy sequence masking: drop tokens with A<0 in sequences whose
    masked mean ``old - new`` exceeds ``opsm_delta``.  Returns ``(mask, clipfrac)``
    where clipfrac sums per-sample ``masked tokens / valid tokens``."""
    seq_kl = masked_seq_mean(old_log_probs - log_probs, loss_mask, seg)
    drop = ((advantages < 0) & (seg.expand(seq_kl) > opsm_delta)).float()
    den = seg.seg_sum(loss_mask.float()).clamp_min(1)
    clipfrac = (seg.seg_sum(drop) / den).sum()
    return 1.0 - drop, clipfrac


# --------------------------------------------------------------------------- policy-gradient losses


def compute_policy_loss(ppo_kl, advantages, eps_clip: float, eps_clip_high: float, eps_clip_c: float | None = None):
    """PPO clipped surrogate with optional dual clip.  ``ppo_kl = old - new``.  On a GPU the whole chain (and its
    gradient) is one kernel; advantages carry no gradient there (they never do in the trainers)."""
    if eps_clip_c is not None and not eps_clip_c > 1.0:
        raise ValueError(f"dual-clip lower bound must be > 1.0, got {eps_clip_c}")
    if ppo_kl.is_cuda and not advantages.requires_grad and ppo_kl.dtype == torch.float32:
        from ..ops import _use_cuda, _cuda

        if _use_cuda(ppo_kl):
            return _cuda().policy_loss(ppo_kl, advantages, eps_clip, eps_clip_high, eps_clip_c)
    ratio = torch.exp(-ppo_kl)
    l1 = -ratio * advantages
    l2 = -ratio.clamp(1.0 - eps_clip, 1.0 + eps_clip_high) * advantages
    clipped = torch.maximum(l1, l2)
    clipfrac = (l2 > l1).float()
    if eps_clip_c is not None:
        if not eps_clip_c > 1.0:
            raise ValueError(f"dual-clip lower bound must be > 1.0, got {eps_clip_c}")
        l3 = -eps_clip_c * advantages
        clipped = torch.where(advantages < 0, torch.minimum(l3, clipped), clipped)
    return clipped, clipfrac


def compute_sapo_loss(ppo_kl, advantages, tau_pos: float, tau_neg: float):
    """Soft gate f(r) = (4/tau) * sigmoid(tau (r-1)); tau depends on sign(A)."""
    ratio = torch.exp(-ppo_kl)
    tau = torch.where(advantages > 0, torch.full_like(advantages, tau_pos), torch.full_like(advantages, tau_neg))
    s = torch.sigmoid(tau * (ratio - 1.0))
    loss = -(4.0 / tau) * s * advantages
    clipfrac = (4.0 * s * (1.0 - s) < 0.9).float()
    return loss, clipfrac


def compute_cispo_loss(log_probs, ppo_kl, advantages, eps_clip: float, eps_clip_high: float):
    """-sg(clip(r)) * sg(A) * logp; the gradient flows through logp only."""
    ratio = torch.exp(-ppo_kl)
    hi, lo = 1.0 + eps_clip_high, 1.0 - eps_clip
    coef = torch.where(advantages >= 0, ratio.clamp(max=hi), ratio.clamp(min=lo))
    loss = -(coef.detach() * advantages.detach() * log_probs)
    clipfrac = ((advantages >= 0) & (ratio > hi)).float() + ((advantages < 0) & (ratio < lo)).float()
    return loss, clipfrac


def compute_rloo_loss(log_probs, advantages):
    """Unclipped REINFORCE term; clipfrac is identically zero."""
    return -(advantages.detach() * log_probs), torch.zeros_like(log_probs)


def _m2po_threshold(sorted_d2: torch.Tensor, target_sum: float) -> tuple[float, float]:
    """Largest |log r| cap tau such that sum(min(d2, tau^2)) <= target_sum."""
    n = sorted_d2.numel()
    total = float(sorted_d2.sum())
    if target_sum >= total - 1e-12:
        return 1e5, total / n
    if target_sum <= 1e-12:
        return 0.0, 0.0
    csum = torch.cumsum(sorted_d2, 0)
    rest = torch.arange(n - 1, -1, -1, device=sorted_d2.device, dtype=sorted_d2.dtype)
    capped = (sorted_d2 - 1e-12) * rest + csum  # total if everything above index k is capped at d2[k]
    hit = torch.nonzero(capped >= target_sum - 1e-12)
    if hit.numel() == 0:
        return 1e5, total / n
    k = int(hit[0])
    if k == 0:
        return 0.0, float(csum[-1]) / n
    prev = float(sorted_d2[k - 1])
    m2_after = (prev * (n - k) + float(csum[k - 1])) / n
    return math.sqrt(max(prev - 1e-12, 0.0)), m2_after


def m2po_clip_bounds(ppo_kl, advantages, kl2_budget: float):
    """Second-moment trust region over 'harmful' tokens (A>0 & r>1, or A<0 & r<1)."""
    ratio = torch.exp(-ppo_kl)
    harmful = ((advantages > 1e-12) & (ratio > 1.0 + 1e-12)) | ((advantages < -1e-12) & (ratio < 1.0 - 1e-12))
    d2 = ppo_kl[harmful].detach().pow(2)
    n = d2.numel()
    if n == 0:
        return 0.0, 1e5, 0.0, 0.0
    m2_now = float(d2.sum()) / n
    if m2_now <= kl2_budget + 1e-12:
        return 0.0, 1e5, m2_now, m2_now
    tau, m2_after = _m2po_threshold(torch.sort(d2).values, kl2_budget * n)
    return math.exp(-tau), math.exp(tau), m2_now, m2_after


def compute_m2po_loss(ppo_kl, advantages, kl2_budget: float, miniclip_low: float = 0.3, miniclip_high: float = 0.5):
    lo, hi, m2_now, m2_after = m2po_clip_bounds(ppo_kl, advantages, kl2_budget)
    eps_low = max(1.0 - lo, miniclip_low)
    eps_high = max(hi - 1.0, miniclip_high)
    ratio = torch.exp(-ppo_kl)
    l1 = -advantages * ratio
    l2 = -advantages * ratio.clamp(1.0 - eps_low, 1.0 + eps_high)
    return torch.maximum(l1, l2), (l2 > l1).float(), m2_now, m2_after, eps_low, eps_high


# --------------------------------------------------------------------------- truncated importance sampling


def vanilla_tis(old_log_probs, rollout_log_probs, tis_clip: float = 2.0, tis_clip_low: float = 0.0):
    """Clamp exp(old - rollout) to [tis_clip_low, tis_clip]; returns (weights, raw ratio, clipfrac)."""
    ois = torch.exp(old_log_probs - rollout_log_probs)
    w = ois.clamp(tis_clip_low, tis_clip)
    return w.detach(), ois.detach(), (w != ois).float()


def icepop_tis(old_log_probs, rollout_log_probs, tis_clip: float = 2.0, tis_clip_low: float = 0.5):
    """IcePop: ratios outside [low, high] are zeroed instead of clamped."""
    ois = torch.exp(old_log_probs - rollout_log_probs)
    inside = (ois >= tis_clip_low) & (ois <= tis_clip)
    w = torch.where(inside, ois, torch.zeros_like(ois))
    return w.detach(), ois.detach(), (~inside).float()


# --------------------------------------------------------------------------- rewards → advantages

GROUP_BASELINE_ALGOS = ("grpo", "gspo", "sapo", "cispo", "m2po", "reinforce_plus_plus_baseline", "rloo")
STD_NORM_ALGOS = ("grpo", "gspo", "sapo", "cispo", "m2po")


def post_process_rewards(
    rewards: torch.Tensor,
    n_samples_per_prompt: int,
    advantage_estimator: str = "grpo",
    rewards_normalization: bool = True,
    grpo_std_normalization: bool = True,
) -> torch.Tensor:
    """Group-wise reward shaping.  ``rewards`` is ordered group-major
    (``[num_groups * n_samples_per_prompt]``).  Returns the shaped rewards."""
    r = rewards.float()
    if not rewards_normalization or advantage_estimator not in GROUP_BASELINE_ALGOS:
        return r
    if r.numel() % n_samples_per_prompt != 0:
        raise ValueError(f"{r.numel()} rewards do not split into groups of {n_samples_per_prompt}")
    g = r.view(-1, n_samples_per_prompt)
    if advantage_estimator == "rloo":
        if n_samples_per_prompt < 2:
            raise ValueError("RLOO needs n_samples_per_prompt >= 2")
        if not torch.isfinite(g).all():
            raise ValueError("RLOO group contains non-finite rewards")
        return ((n_samples_per_prompt / (n_samples_per_prompt - 1)) * (g - g.mean(-1, keepdim=True))).reshape(-1)
    g = g - g.mean(-1, keepdim=True)
    if advantage_estimator in STD_NORM_ALGOS and grpo_std_normalization:
        std = g.std(-1, keepdim=True) if n_samples_per_prompt > 1 else torch.zeros_like(g)
        g = g / (std + 1e-6)
    return g.reshape(-1)


def get_grpo_returns(rewards: torch.Tensor, seg: Segments) -> torch.Tensor:
    """Broadcast each sample's scalar over its response tokens."""
    return seg.expand(rewards.float())


def get_reinforce_plus_plus_returns(rewards, kl, loss_mask, seg: Segments, kl_coef: float, gamma: float):
    """Discounted return-to-go with token reward ``-kl_coef * kl`` and the scalar
    reward added at the last valid token of each sample; masked tokens return 0."""
    valid = loss_mask != 0
    r = torch.where(valid, -kl_coef * kl.float(), torch.zeros_like(kl, dtype=torch.float32))
    cu = seg.cu
    # index of the last valid token per sample (samples without any valid token get none)
    pos = torch.arange(r.numel(), device=r.device)
    last = torch.full((seg.num,), -1, dtype=torch.int64, device=r.device)
    last = last.scatter_reduce(0, seg.ids[valid], pos[valid], reduce="amax", include_self=True)
    has = last >= 0
    r = r.index_add(0, last[has], rewards.float().to(r.device)[has])
    out = _segmented_discounted_suffix_sum(r, seg, gamma)
    return torch.where(valid, out, torch.zeros_like(out))


def _segmented_discounted_suffix_sum(x: torch.Tensor, seg: Segments, gamma: float) -> torch.Tensor:
    """y[t] = x[t] + gamma * y[t+1] inside each segment."""
    if x.numel() == 0:
        return x
    lens = seg.lengths.tolist()
    L = max(lens) if lens else 0
    B = len(lens)
    pad = x.new_zeros(B, L)
    idx_in = torch.arange(x.numel(), device=x.device) - seg.expand(seg.cu[:-1])
    pad[seg.ids, idx_in] = x
    if gamma == 1.0:
        y = torch.flip(torch.cumsum(torch.flip(pad, [1]), 1), [1])
    else:
        y = torch.zeros_like(pad)
        run = x.new_zeros(B)
        for t in range(L - 1, -1, -1):
            run = pad[:, t] + gamma * run
            y[:, t] = run
    return y[seg.ids, idx_in]


def vanilla_gae(rewards_tok, values, seg: Segments, gamma: float, lambd: float):
    """Generalised advantage estimation on packed per-token rewards/values.
    Returns (advantages, returns)."""
    lens = seg.lengths.tolist()
    B, L = len(lens), (max(lens) if lens else 0)
    idx_in = torch.arange(values.numel(), device=values.device) - seg.expand(seg.cu[:-1])
    v = values.new_zeros(B, L + 1).float()
    r = values.new_zeros(B, L).float()
    v[seg.ids, idx_in] = values.float()
    r[seg.ids, idx_in] = rewards_tok.float()
    adv = torch.zeros_like(r)
    last = r.new_zeros(B)
    for t in range(L - 1, -1, -1):
        delta = r[:, t] + gamma * v[:, t + 1] - v[:, t]
        last = delta + gamma * lambd * last
        adv[:, t] = last
    ret = adv + v[:, :L]
    return adv[seg.ids, idx_in], ret[seg.ids, idx_in]


def chunked_gae(rewards_tok, values, seg: Segments, gamma: float, lambd: float, chunk: int = 128):
    """GAE evaluated as a blocked linear recurrence: inside a chunk the scan is a
    triangular mat-vec, chunks are chained by their carry.  Same result as
    :func:`vanilla_gae` with O(L/chunk) sequential steps."""
    lens = seg.lengths.tolist()
    B, L = len(lens), (max(lens) if lens else 0)
    if L == 0:
        return values.float(), values.float()
    idx_in = torch.arange(values.numel(), device=values.device) - seg.expand(seg.cu[:-1])
    v = values.new_zeros(B, L + 1).float()
    r = values.new_zeros(B, L).float()
    v[seg.ids, idx_in] = values.float()
    r[seg.ids, idx_in] = rewards_tok.float()
    delta = r + gamma * v[:, 1:] - v[:, :-1]
    w = gamma * lambd
    adv = torch.zeros_like(delta)
    carry = delta.new_zeros(B)
    n_chunks = (L + chunk - 1) // chunk
    k = torch.arange(chunk, device=delta.device)
    # M[i, j] = w^(j-i) for j >= i
    expo = (k[None, :] - k[:, None]).clamp_min(0).float()
    M = torch.where(k[None, :] >= k[:, None], torch.pow(torch.tensor(w, device=delta.device), expo), torch.zeros(()))
    for c in range(n_chunks - 1, -1, -1):
        s, e = c * chunk, min(L, (c + 1) * chunk)
        n = e - s
        blk = delta[:, s:e] @ M[:n, :n].T
        tail = torch.pow(torch.tensor(w, device=delta.device), (n - k[:n]).float())
        blk = blk + carry[:, None] * tail[None, :]
        adv[:, s:e] = blk
        carry = blk[:, 0]
    ret = adv + v[:, :L]
    return adv[seg.ids, idx_in], ret[seg.ids, idx_in]


def ppo_token_rewards(rewards, kl, loss_mask, seg: Segments, kl_coef: float):
    """Token rewards for PPO/GAE: ``-kl_coef*kl`` everywhere plus the scalar
    reward on the last token of each response."""
    r = -kl_coef * kl.float()
    last_idx = seg.cu[1:] - 1
    ok = seg.lengths > 0
    return r.index_add(0, last_idx[ok], rewards.float().to(r.device)[ok])


# --------------------------------------------------------------------------- whitening


def masked_whiten(x, mask, shift_mean: bool = True, group=None, eps: float = 1e-8):
    """(x - mean) / sqrt(var + eps) with statistics over masked entries; when a
    process group is given the three sums are all-reduced over it."""
    import torch.distributed as dist

    m = mask.to(x.dtype)
    stats = torch.stack([(x * m).sum(), (x * x * m).sum(), m.sum()])
    if group is not None and dist.is_initialized():
        dist.all_reduce(stats, group=group)
    s1, s2, n = stats.unbind()
    n = n.clamp_min(1)
    mean = s1 / n
    var = (s2 / n - mean * mean).clamp_min(0)
    # Bessel's correction, as the distributed reference statistic uses
    var = var * n / (n - 1).clamp_min(1)
    out = (x - mean) * torch.rsqrt(var + eps)
    if not shift_mean:
        out = out + mean
    return out


def masked_normalize(x, mask, group=None, variance_floor: float = 1e-8, return_stats: bool = False):
    """REINFORCE++ advantage normalisation (relax/utils/distributed_utils.py distributed_masked_normalize
    :161-213): mean and POPULATION variance (ddof = 0) over every mask-nonzero element of the whole
    data-parallel group, ``(x - mean) * rsqrt(max(var, floor))`` inside the mask and exactly zero outside.
    With ``return_stats`` also returns ``{raw_mean, raw_std, normalized_mean, normalized_std, valid_token_count,
    zero_variance}`` as the reference logs them (relax/backends/megatron/loss.py:706-726)."""
    import torch.distributed as dist

    if variance_floor <= 0:
        raise ValueError("variance_floor must be positive")
    wd = torch.float64 if x.dtype == torch.float64 else torch.float32
    xv = x.to(wd)
    valid = mask != 0
    m = valid.to(wd)
    s = torch.stack([torch.where(valid, xv, torch.zeros_like(xv)).sum(), m.sum()])
    if group is not None and dist.is_initialized():
        dist.all_reduce(s, group=group)
    cnt = s[1].clamp_min(1)
    mean = s[0] / cnt
    c = torch.where(valid, xv - mean, torch.zeros_like(xv))
    v = c.square().sum().reshape(1)
    if group is not None and dist.is_initialized():
        dist.all_reduce(v, group=group)
    var = (v[0] / cnt).clamp_min(0.0)
    out = torch.where(valid, (xv - mean) * torch.rsqrt(var.clamp_min(variance_floor)), torch.zeros_like(xv)).to(x.dtype)
    if not return_stats:
        return out
    nvar = var / torch.maximum(var, torch.tensor(variance_floor, dtype=wd, device=x.device))
    stats = {"reinforce_pp_advantage_raw_mean": mean.detach(), "reinforce_pp_advantage_raw_std": var.sqrt().detach(),
             "reinforce_pp_advantage_normalized_mean": torch.zeros_like(mean), "reinforce_pp_advantage_normalized_std": nvar.sqrt().detach(),
             "reinforce_pp_valid_token_count": s[1].detach(), "reinforce_pp_zero_variance": (var == 0).to(wd).detach()}
    return out, stats
