"""Loss functions of the trainer, on packed response-token streams.

A micro-batch is described by :class:`LossBatch`: flat fp32 tensors over all
response tokens that live on this rank (after context-parallel slicing) plus
the :class:`~relax_b200.algo.ppo_utils.Segments` that split them per sample.
Parity targets: relax/backends/megatron/loss.py:824-1185 (policy loss),
:1188-1244 (value loss), :1247-1298 (SFT), :1443-1620 (dispatcher + scaling);
relax/backends/megatron/cp_utils.py:125-206 (reducers).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from . import ppo_utils as P
from .ppo_utils import Segments


@dataclass
class LossConfig:
    advantage_estimator: str = "grpo"
    eps_clip: float = 0.2
    eps_clip_high: Optional[float] = None
    eps_clip_c: Optional[float] = None
    entropy_coef: float = 0.0
    use_kl_loss: bool = False
    kl_loss_coef: float = 0.0
    kl_loss_type: str = "k1"
    use_unbiased_kl: bool = False
    # on-policy distillation as a loss term (the teacher's log-probs of the sampled tokens travel in LossBatch.extras)
    opd_loss_coef: float = 0.0
    opd_kl_type: str = "reverse_kl"
    opd_per_token_clip: Optional[float] = None
    opd_is_clip: Optional[float] = None
    opd_log_prob_min_clamp: Optional[float] = None
    use_tis: bool = False
    tis_clip: float = 2.0
    tis_clip_low: float = 0.0
    tis_mode: str = "vanilla"  # vanilla | icepop
    get_mismatch_metrics: bool = False
    use_opsm: bool = False
    opsm_delta: float = 1e-4
    calculate_per_token_loss: bool = False
    sapo_tau_pos: float = 1.0
    sapo_tau_neg: float = 1.05
    m2po_kl2_budget: float = 0.04
    m2po_miniclip_low: float = 0.3
    m2po_miniclip_high: float = 0.5
    true_on_policy: bool = False
    value_clip: float = 0.2
    custom_pg_loss_reducer: Optional[Callable] = None
    custom_tis_function: Optional[Callable] = None
    # fn(log_probs, entropy, LossBatch, LossConfig) -> (loss, metrics): replaces the policy loss (--loss-type custom_loss)
    custom_loss_function: Optional[Callable] = None

    def __post_init__(self):
        if self.eps_clip_high is None:
            self.eps_clip_high = self.eps_clip

    @staticmethod
    def from_args(args) -> "LossConfig":
        kw = {}
        for f in LossConfig.__dataclass_fields__:
            if hasattr(args, f):
                kw[f] = getattr(args, f)
        from ..rollout.custom_generate import load_function

        # --custom-*-function-path flags name user code ("pkg.mod:fn" or "/file.py:fn")
        for field_name, flag, npos in (("custom_tis_function", "custom_tis_function_path", 3),
                                       ("custom_pg_loss_reducer", "custom_pg_loss_reducer_function_path", 3),
                                       ("custom_loss_function", "custom_loss_function_path", 4)):
            path = getattr(args, flag, None)
            if path:
                kw[field_name] = load_function(path, npos, flag)
        return LossConfig(**kw)


@dataclass
class LossBatch:
    seg: Segments                      # local response tokens per sample
    loss_mask: torch.Tensor            # [T] float
    advantages: Optional[torch.Tensor] = None
    old_log_probs: Optional[torch.Tensor] = None
    ref_log_probs: Optional[torch.Tensor] = None
    rollout_log_probs: Optional[torch.Tensor] = None
    returns: Optional[torch.Tensor] = None
    values: Optional[torch.Tensor] = None
    # denominators of the per-sample mean; defaults to the full-sample mask sums.
    # Under context parallelism they are the FULL sample's mask sums (so shards add up),
    # and multi-turn samples split over rows share ``sample_index_mask_sums``.
    sample_denoms: Optional[torch.Tensor] = None
    # full (un-sliced) tensors for sequence-level quantities under CP
    full_seg: Optional[Segments] = None
    gather_full: Optional[Callable[[torch.Tensor], torch.Tensor]] = None
    full_loss_mask: Optional[torch.Tensor] = None
    extras: dict = field(default_factory=dict)


def make_reducer(seg: Segments, loss_mask: torch.Tensor, per_token: bool, sample_denoms=None):
    """Return ``f(x[T]) -> scalar``.

    Default: sum over samples of the per-sample masked mean (denominator clamped
    to >= 1).  ``per_token``: plain masked sum, normalised later by the global
    token count."""
    m = loss_mask.float()
    if per_token:
        return lambda x: (x * m).sum()
    den = (sample_denoms.float() if sample_denoms is not None else seg.seg_sum(m)).clamp_min(1)

    def red(x):
        return (seg.seg_sum(x * m) / den).sum()

    return red


def policy_loss(log_probs: torch.Tensor, entropy: torch.Tensor, b: LossBatch, cfg: LossConfig):
    """Returns ``(loss, metrics)``; all reductions are 'sum of sample means'
    (or token sums) - the caller applies the global scaling."""
    seg = b.seg
    red = make_reducer(seg, b.loss_mask, cfg.calculate_per_token_loss, b.sample_denoms)
    adv = b.advantages
    old = log_probs.detach() if (cfg.true_on_policy or b.old_log_probs is None) else b.old_log_probs

    need_full = cfg.use_opsm or cfg.advantage_estimator == "gspo"
    if need_full:
        gather = b.gather_full or (lambda x: x)
        fseg = b.full_seg or seg
        fmask = b.full_loss_mask if b.full_loss_mask is not None else b.loss_mask
        full_lp, full_old = gather(log_probs), gather(old)

    metrics = {}
    if cfg.use_opsm:
        full_adv = (b.gather_full or (lambda x: x))(adv)
        opsm_full, opsm_clipfrac = P.compute_opsm_mask(full_lp, full_old, full_adv, fmask, fseg, cfg.opsm_delta)
        slicer = b.extras.get("slice_local", lambda x: x)
        opsm_mask = slicer(opsm_full)
        metrics["opsm_clipfrac"] = opsm_clipfrac.detach()

    if cfg.advantage_estimator == "gspo":
        ppo_kl = P.compute_gspo_kl(full_lp, full_old, fmask, fseg, expand_seg=seg)
    else:
        ppo_kl = old - log_probs

    est = cfg.advantage_estimator
    if est == "sapo":
        pg, clipfrac = P.compute_sapo_loss(ppo_kl, adv, cfg.sapo_tau_pos, cfg.sapo_tau_neg)
    elif est == "cispo":
        pg, clipfrac = P.compute_cispo_loss(log_probs, ppo_kl, adv, cfg.eps_clip, cfg.eps_clip_high)
    elif est == "m2po":
        pg, clipfrac, m2n, m2a, el, eh = P.compute_m2po_loss(
            ppo_kl, adv, cfg.m2po_kl2_budget, cfg.m2po_miniclip_low, cfg.m2po_miniclip_high
        )
        dev = ppo_kl.device
        metrics.update(
            ppo_kl_m2_before=torch.tensor(m2n, device=dev), ppo_kl_m2_after=torch.tensor(m2a, device=dev),
            m2po_eps_low=torch.tensor(el, device=dev), m2po_eps_high=torch.tensor(eh, device=dev),
        )
    elif est == "rloo":
        pg, clipfrac = P.compute_rloo_loss(log_probs, adv)
    else:
        pg, clipfrac = P.compute_policy_loss(ppo_kl, adv, cfg.eps_clip, cfg.eps_clip_high, cfg.eps_clip_c)

    if cfg.use_opsm:
        pg = pg * opsm_mask

    pg_red = red
    if cfg.use_tis or cfg.get_mismatch_metrics:
        if b.rollout_log_probs is None:
            raise ValueError("rollout_log_probs are required for TIS / mismatch metrics")
        if cfg.custom_tis_function is not None:
            w, ois_raw, tclip = cfg.custom_tis_function(old, b.rollout_log_probs, cfg)
        elif cfg.tis_mode == "icepop":
            w, ois_raw, tclip = P.icepop_tis(old, b.rollout_log_probs, cfg.tis_clip, cfg.tis_clip_low)
        else:
            w, ois_raw, tclip = P.vanilla_tis(old, b.rollout_log_probs, cfg.tis_clip, cfg.tis_clip_low)
        metrics["ois"] = red(torch.exp(-ppo_kl)).detach()
        metrics["tis"] = red(ois_raw).detach()
        metrics["tis_clipfrac"] = red(tclip).detach()
        if cfg.use_tis:
            pg = pg * w
    if cfg.custom_pg_loss_reducer is not None:
        pg_red = cfg.custom_pg_loss_reducer(seg, b.loss_mask, cfg.calculate_per_token_loss)

    pg_loss = pg_red(pg)
    pg_clipfrac = red(clipfrac)
    ppo_kl_m = red(ppo_kl)
    entropy_loss = red(entropy)
    loss = pg_loss - cfg.entropy_coef * entropy_loss

    if cfg.use_kl_loss:
        if b.ref_log_probs is None:
            raise ValueError("use_kl_loss needs ref_log_probs")
        ir = torch.exp(log_probs - old).detach() if cfg.use_unbiased_kl else None
        kl = P.compute_approx_kl(log_probs, b.ref_log_probs, cfg.kl_loss_type, ir)
        kl_loss = red(kl)
        loss = loss + cfg.kl_loss_coef * kl_loss
        metrics["kl_loss"] = kl_loss.detach()

    if cfg.opd_loss_coef != 0.0 and b.extras.get("teacher_log_probs") is not None:
        # on-policy distillation as a differentiable loss term (relax/utils/opd/opd_utils.py compute_policy_opd_loss
        # :1366-1455): per-token divergence of the sampled token, clipped from above, optionally weighted by the
        # truncated importance ratio of the current to the old policy
        from . import opd as _opd

        d = _opd.token_kl(log_probs, b.extras["teacher_log_probs"].detach(), kl_type=cfg.opd_kl_type,
                          log_prob_min_clamp=cfg.opd_log_prob_min_clamp)
        if cfg.opd_per_token_clip is not None:
            metrics["opd_per_token_clip_frac"] = red((d > cfg.opd_per_token_clip).float()).detach()
            d = d.clamp(max=float(cfg.opd_per_token_clip))
        if cfg.opd_is_clip is not None:
            ratio = torch.exp(log_probs.detach() - old.detach())
            metrics["opd_is_clip_frac"] = red((ratio > cfg.opd_is_clip).float()).detach()
            d = d * ratio.clamp(max=float(cfg.opd_is_clip))
        opd_l = red(d)
        loss = loss + cfg.opd_loss_coef * opd_l
        metrics["opd_loss"] = opd_l.detach()

    if log_probs.numel() == 0:
        loss = loss + 0.0 * log_probs.sum()

    if b.rollout_log_probs is not None:
        metrics["train_rollout_logprob_abs_diff"] = red((old - b.rollout_log_probs).abs()).detach()
        metrics["train_rollout_prob_abs_diff"] = red((old.exp() - b.rollout_log_probs.exp()).abs()).detach()

    metrics.update(
        loss=loss.detach(), pg_loss=pg_loss.detach(), entropy_loss=entropy_loss.detach(),
        pg_clipfrac=pg_clipfrac.detach(), ppo_kl=ppo_kl_m.detach(),
    )
    return loss, metrics


def value_loss(values: torch.Tensor, b: LossBatch, cfg: LossConfig):
    """Clipped value loss: max((v-R)^2, (clip(v, old±c)-R)^2) (no 1/2 factor)."""
    red = make_reducer(b.seg, b.loss_mask, cfg.calculate_per_token_loss, b.sample_denoms)
    old_v, ret = b.values, b.returns
    v_clip = old_v + (values - old_v).clamp(-cfg.value_clip, cfg.value_clip)
    l1 = (v_clip - ret) ** 2
    l2 = (values - ret) ** 2
    vloss = red(torch.maximum(l1, l2))
    clipfrac = red((l1 > l2).float())
    if values.numel() == 0:
        vloss = vloss + 0.0 * values.sum()
    return vloss, {"value_loss": vloss.detach(), "value_clipfrac": clipfrac.detach()}


def sft_loss(log_probs: torch.Tensor, b: LossBatch, cfg: LossConfig):
    red = make_reducer(b.seg, b.loss_mask, cfg.calculate_per_token_loss, b.sample_denoms)
    loss = red(-log_probs)
    if log_probs.numel() == 0:
        loss = loss + 0.0 * log_probs.sum()
    return loss, {"loss": loss.detach()}


def seq_cls_loss(logits: torch.Tensor, labels: torch.Tensor, problem_type: str = "single_label_classification",
                 threshold: float = 0.5):
    """Sum over samples of the classification loss (the caller divides by the global batch size, as for the other
    per-sample losses) and the number of correct predictions (relax/backends/megatron/loss.py :1301-1383).
    ``single_label_classification``: ``labels [n]`` class ids, cross entropy, accuracy by arg-max.
    ``multi_label_classification``: ``labels [n, C]`` multi-hot, mean binary cross entropy over the classes of each
    sample, ``accuracy`` counts samples whose thresholded sigmoid matches every label, ``label_accuracy`` the mean
    per-label agreement."""
    if problem_type == "multi_label_classification":
        y = labels.to(logits.device).float()
        bce = torch.nn.functional.binary_cross_entropy_with_logits(logits.float(), y, reduction="none").mean(-1).sum()
        pred = (torch.sigmoid(logits.float()) > threshold).float()
        agree = (pred == y).float()
        return bce, {"loss": bce.detach(), "accuracy": agree.min(-1).values.sum(), "label_accuracy": agree.mean(-1).sum()}
    if problem_type not in ("single_label_classification", None):
        raise ValueError(f"unknown problem type {problem_type!r}")
    ce = torch.nn.functional.cross_entropy(logits.float(), labels.long(), reduction="sum")
    acc = (logits.argmax(-1) == labels).float().sum()
    return ce, {"loss": ce.detach(), "accuracy": acc}


def scale_loss(loss, *, per_token: bool, num_microbatches: int, global_batch_size: int, dp_cp_world: int,
               num_tokens: Optional[torch.Tensor] = None, is_dummy: bool = False, explicit_scale: Optional[float] = None):
    """Scaling applied before backward so that the gradient AVERAGE over the
    dp x cp world equals the gradient of the mean over ``global_batch_size``
    samples (relax/backends/megatron/loss.py:1562-1596).  Dummy micro-batches
    contribute ``0 * loss`` so every rank runs the same number of backward
    passes."""
    if is_dummy:
        return loss * 0.0
    if explicit_scale is not None:
        return loss * explicit_scale
    if per_token:
        # caller divides by the all-reduced token count after accumulation
        return loss
    return loss * (num_microbatches / global_batch_size * dp_cp_world) / num_microbatches


def compute_advantages_and_returns(
    estimator: str,
    rewards: torch.Tensor,
    seg: Segments,
    loss_mask: torch.Tensor,
    *,
    log_probs: Optional[torch.Tensor] = None,
    ref_log_probs: Optional[torch.Tensor] = None,
    values: Optional[torch.Tensor] = None,
    kl_coef: float = 0.0,
    kl_loss_type: str = "k1",
    gamma: float = 1.0,
    lambd: float = 1.0,
    normalize_advantages: bool = False,
    dp_group=None,
    custom_advantage: Optional[torch.Tensor] = None,
    stats_out: Optional[dict] = None,
):
    """Advantage/return estimation for all supported estimators
    (relax/backends/megatron/loss.py:532-738).  ``rewards`` are the already
    group-shaped scalars (see :func:`ppo_utils.post_process_rewards`)."""
    T = int(seg.lengths.sum())
    dev = loss_mask.device
    if log_probs is not None and ref_log_probs is not None:
        kl = P.compute_approx_kl(log_probs, ref_log_probs, kl_loss_type)
    else:
        kl = torch.zeros(T, device=dev)

    if custom_advantage is not None:
        adv = seg.expand(custom_advantage.float())
        ret = adv
    elif estimator in ("grpo", "gspo", "sapo", "cispo", "m2po", "rloo"):
        adv = P.get_grpo_returns(rewards.to(dev), seg)
        ret = adv
    elif estimator == "reinforce_plus_plus":
        ret = P.get_reinforce_plus_plus_returns(rewards.to(dev), kl, loss_mask, seg, kl_coef, gamma)
        adv = ret
    elif estimator == "reinforce_plus_plus_baseline":
        adv = torch.where(loss_mask != 0, seg.expand(rewards.float().to(dev)), torch.zeros(T, device=dev))
        ret = adv
    elif estimator == "ppo":
        if values is None:
            raise ValueError("ppo needs critic values")
        r_tok = P.ppo_token_rewards(rewards.to(dev), kl, loss_mask, seg, kl_coef)
        adv, ret = P.chunked_gae(r_tok, values, seg, gamma, lambd)
    else:
        raise ValueError(f"unknown advantage estimator {estimator}")

    if normalize_advantages:
        if estimator in ("reinforce_plus_plus", "reinforce_plus_plus_baseline"):
            # population moments with a variance floor, not the Bessel-corrected whitening of the other estimators
            adv, st = P.masked_normalize(adv, loss_mask, group=dp_group, return_stats=True)
            if stats_out is not None:
                stats_out.update(st)
        else:
            adv = P.masked_whiten(adv, loss_mask, group=dp_group) * (loss_mask != 0)
    return adv, ret
