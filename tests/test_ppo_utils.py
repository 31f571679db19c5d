import math

import pytest
import torch

from relax_b200.algo import ppo_utils as P
from relax_b200.algo.ppo_utils import Segments


def test_kl_estimators():
    a, b = torch.tensor([-1.0, -2.0, -0.5]), torch.tensor([-1.5, -1.0, -0.5])
    d = a - b
    assert torch.allclose(P.compute_approx_kl(a, b, "k1"), d)
    assert torch.allclose(P.compute_approx_kl(a, b, "k2"), d * d / 2)
    k3 = torch.exp(-d) - 1 + d
    assert torch.allclose(P.compute_approx_kl(a, b, "k3"), k3)
    big = P.compute_approx_kl(torch.tensor([-30.0]), torch.tensor([0.0]), "low_var_kl")
    assert big.item() == 10.0
    ir = torch.tensor([2.0, 1.0, 0.5])
    assert torch.allclose(P.compute_approx_kl(a, b, "k3", ir), k3 * ir)
    with pytest.raises(ValueError):
        P.compute_approx_kl(a, b, "nope")


def test_ppo_clip_and_dual_clip():
    kl = torch.tensor([0.0, -0.5, 0.5, -2.0])   # ratio = exp(-kl)
    adv = torch.tensor([1.0, 1.0, -1.0, -1.0])
    loss, cf = P.compute_policy_loss(kl, adv, 0.2, 0.2)
    r = torch.exp(-kl)
    exp = torch.maximum(-r * adv, -r.clamp(0.8, 1.2) * adv)
    assert torch.allclose(loss, exp)
    assert cf.tolist() == [0.0, 1.0, 1.0, 0.0]
    loss2, _ = P.compute_policy_loss(kl, adv, 0.2, 0.2, eps_clip_c=3.0)
    assert loss2[3].item() == pytest.approx(3.0)      # -c * A caps the negative-advantage branch
    assert loss2[0].item() == loss[0].item()
    with pytest.raises(ValueError):
        P.compute_policy_loss(kl, adv, 0.2, 0.2, eps_clip_c=0.5)


def test_sapo_on_policy_value_and_grad():
    kl = torch.zeros(4, requires_grad=True)
    adv = torch.tensor([1.0, -1.0, 2.0, -0.5])
    loss, cf = P.compute_sapo_loss(kl, adv, 1.0, 1.05)
    tau = torch.tensor([1.0, 1.05, 1.0, 1.05])
    assert torch.allclose(loss, -(2.0 / tau) * adv)
    assert cf.sum() == 0
    loss.sum().backward()
    # d/d(kl) of -(4/tau) sigmoid(tau (e^{-kl} - 1)) A at kl=0 = A   (gate slope 1 at r=1)
    assert torch.allclose(kl.grad, adv, atol=1e-6)


def test_cispo_and_rloo_gradient_paths():
    lp = torch.tensor([-1.0, -1.2, -0.3], requires_grad=True)
    old = torch.tensor([-1.1, -0.2, -0.3])
    adv = torch.tensor([1.0, -1.0, 0.5])
    loss, cf = P.compute_cispo_loss(lp, old - lp, adv, 0.2, 0.2)
    loss.sum().backward()
    ratio = torch.exp(lp.detach() - old)
    coef = torch.where(adv >= 0, ratio.clamp(max=1.2), ratio.clamp(min=0.8))
    assert torch.allclose(lp.grad, -coef * adv)
    assert cf.tolist() == [0.0, 1.0, 0.0]
    lp2 = lp.detach().clone().requires_grad_()
    l2, c2 = P.compute_rloo_loss(lp2, adv)
    l2.sum().backward()
    assert torch.allclose(lp2.grad, -adv) and c2.sum() == 0


def test_m2po_threshold_bruteforce():
    torch.manual_seed(0)
    kl = torch.randn(200) * 0.5
    adv = torch.randn(200)
    budget = 0.02
    lo, hi, m2n, m2a = P.m2po_clip_bounds(kl, adv, budget)
    assert m2n > budget and m2a <= budget + 1e-6
    assert lo == pytest.approx(1.0 / hi)
    # nothing harmful -> open bounds
    lo2, hi2, _, _ = P.m2po_clip_bounds(torch.zeros(4), torch.ones(4), budget)
    assert lo2 == 0.0 and hi2 == 1e5
    loss, cf, *_ = P.compute_m2po_loss(kl, adv, budget)
    assert loss.shape == kl.shape and cf.max() <= 1


def test_tis_variants():
    old, ro = torch.tensor([0.0, 1.0, -3.0]), torch.tensor([0.0, 0.0, 0.0])
    w, raw, c = P.vanilla_tis(old, ro, 2.0, 0.1)
    assert torch.allclose(w, torch.tensor([1.0, 2.0, 0.1])) and c.tolist() == [0.0, 1.0, 1.0]
    w, raw, c = P.icepop_tis(old, ro, 2.0, 0.5)
    assert w.tolist() == [1.0, 0.0, 0.0]


def test_post_process_rewards():
    r = torch.tensor([1.0, 0.0, 0.0, 1.0, 2.0, 2.0, 2.0, 2.0])
    out = P.post_process_rewards(r, 4, "grpo")
    g = r.view(2, 4)
    exp = (g - g.mean(-1, keepdim=True)) / (g.std(-1, keepdim=True) + 1e-6)
    assert torch.allclose(out.view(2, 4), exp)
    assert out[4:].abs().max() == 0
    out = P.post_process_rewards(r, 4, "rloo")
    assert torch.allclose(out[:4], (4 / 3) * (r[:4] - 0.5))
    out = P.post_process_rewards(r, 4, "reinforce_plus_plus_baseline")
    assert torch.allclose(out[:4], r[:4] - 0.5)          # no std division
    assert torch.equal(P.post_process_rewards(r, 4, "ppo"), r)
    with pytest.raises(ValueError):
        P.post_process_rewards(r[:7], 4, "grpo")
    with pytest.raises(ValueError):
        P.post_process_rewards(torch.tensor([1.0]), 1, "rloo")


def test_reinforce_pp_returns_vs_loop():
    torch.manual_seed(1)
    lens = [5, 3, 4]
    seg = Segments.from_lengths(lens)
    kl = torch.randn(sum(lens))
    mask = torch.tensor([1, 1, 1, 0, 0, 1, 1, 1, 0, 0, 0, 0.0])
    rewards = torch.tensor([1.0, -2.0, 3.0])
    for gamma in (1.0, 0.9):
        out = P.get_reinforce_plus_plus_returns(rewards, kl, mask, seg, 0.1, gamma)
        exp, o = [], 0
        for i, L in enumerate(lens):
            m, k = mask[o:o + L], kl[o:o + L]
            valid = m != 0
            if not valid.any():
                exp.append(torch.zeros(L))
            else:
                tr = torch.where(valid, -0.1 * k, torch.zeros(L))
                tr[valid.nonzero()[-1, 0]] += rewards[i]
                ret, run = torch.zeros(L), 0.0
                for t in reversed(range(L)):
                    run = tr[t] + gamma * run
                    ret[t] = run
                exp.append(torch.where(valid, ret, torch.zeros(L)))
            o += L
        assert torch.allclose(out, torch.cat(exp), atol=1e-6)


@pytest.mark.parametrize("gamma,lambd", [(1.0, 1.0), (0.99, 0.95)])
def test_gae_chunked_equals_vanilla(gamma, lambd):
    torch.manual_seed(2)
    lens = [300, 17, 129]
    seg = Segments.from_lengths(lens)
    r, v = torch.randn(sum(lens)) * 0.1, torch.randn(sum(lens))
    a1, r1 = P.vanilla_gae(r, v, seg, gamma, lambd)
    a2, r2 = P.chunked_gae(r, v, seg, gamma, lambd, chunk=64)
    assert torch.allclose(a1, a2, atol=1e-4) and torch.allclose(r1, r2, atol=1e-4)
    # hand check on the shortest segment
    s = 300
    adv, last = torch.zeros(17), 0.0
    for t in reversed(range(17)):
        nv = v[s + t + 1] if t < 16 else 0.0
        last = r[s + t] + gamma * nv - v[s + t] + gamma * lambd * last
        adv[t] = last
    assert torch.allclose(a1[s:s + 17], adv, atol=1e-5)


def test_gspo_and_opsm():
    seg = Segments.from_lengths([2, 3])
    lp = torch.tensor([-1.0, -2.0, -1.0, -1.0, -1.0])
    old = torch.tensor([-1.5, -1.5, -1.0, -2.0, -3.0])
    mask = torch.tensor([1.0, 1, 1, 1, 0])
    kl = P.compute_gspo_kl(lp, old, mask, seg)
    assert torch.allclose(kl, torch.tensor([0.0, 0.0, -0.5, -0.5, -0.5]))
    adv = torch.tensor([-1.0, -1.0, 1.0, -1.0, -1.0])
    m, cf = P.compute_opsm_mask(lp, old + 1.0, adv, mask, seg, 0.2)
    # seq0 kl = 1.0 > delta, negative advantages dropped; seq1 kl = 0.5 > delta
    assert m.tolist() == [0.0, 0.0, 1.0, 0.0, 0.0]


def test_masked_whiten():
    x = torch.tensor([1.0, 2.0, 3.0, 100.0])
    m = torch.tensor([1.0, 1.0, 1.0, 0.0])
    w = P.masked_whiten(x, m)
    assert w[:3].mean().abs() < 1e-6
    assert torch.allclose(w[:3].std(), torch.tensor(1.0), atol=1e-3)


def test_reinforce_pp_normalisation_uses_population_moments_and_reports_stats():
    """REINFORCE++ advantages: (x - mean) * rsqrt(max(var_pop, 1e-8)) inside the mask, 0 outside; zero variance
    maps to zeros and is flagged (relax/utils/distributed_utils.py:161-213)."""
    from relax_b200.algo import loss as L
    from relax_b200.algo import ppo_utils as P
    from relax_b200.algo.ppo_utils import Segments

    x = torch.tensor([1.0, 2.0, 4.0, 100.0, 7.0])
    mask = torch.tensor([1.0, 1.0, 1.0, 0.0, 1.0])
    out, st = P.masked_normalize(x, mask, return_stats=True)
    v = x[mask != 0]
    mean, var = v.mean(), v.var(unbiased=False)
    exp = torch.where(mask != 0, (x - mean) / var.sqrt(), torch.zeros_like(x))
    assert torch.allclose(out, exp, atol=1e-6) and out[3] == 0
    assert abs(float(st["reinforce_pp_advantage_raw_mean"]) - float(mean)) < 1e-6
    assert abs(float(st["reinforce_pp_advantage_raw_std"]) - float(var.sqrt())) < 1e-6
    assert float(st["reinforce_pp_valid_token_count"]) == 4 and float(st["reinforce_pp_zero_variance"]) == 0
    assert abs(float(st["reinforce_pp_advantage_normalized_std"]) - 1.0) < 1e-6
    # differs from the Bessel-corrected whitening used for the other estimators
    assert not torch.allclose(out, P.masked_whiten(x, mask) * (mask != 0), atol=1e-3)
    # zero variance: zeros, flagged, no NaN
    out0, st0 = P.masked_normalize(torch.full((4,), 3.0), torch.ones(4), return_stats=True)
    assert torch.equal(out0, torch.zeros(4)) and float(st0["reinforce_pp_zero_variance"]) == 1
    assert float(st0["reinforce_pp_advantage_normalized_std"]) == 0
    # dispatch inside compute_advantages_and_returns
    seg = Segments.from_lengths([3, 2])
    stats = {}
    adv, _ = L.compute_advantages_and_returns("reinforce_plus_plus_baseline", torch.tensor([1.0, -1.0]), seg, torch.ones(5),
                                             normalize_advantages=True, stats_out=stats)
    raw = torch.tensor([1.0, 1.0, 1.0, -1.0, -1.0])
    assert torch.allclose(adv, (raw - raw.mean()) / raw.var(unbiased=False).sqrt(), atol=1e-6)
    assert "reinforce_pp_advantage_raw_std" in stats


def test_use_rollout_entropy_adds_entropies_to_the_rollout_data():
    """``--use-rollout-entropy``: the forward-only actor and reference passes also return per-token entropies; they
    travel with the batch and show up in the rollout summary."""
    import torch

    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    actor = TrainActor(get_config("tiny"), TrainConfig(n_samples_per_prompt=2, global_batch_size=4, max_tokens_per_gpu=512,
                                                       use_rollout_entropy=True, loss=LossConfig(use_kl_loss=True, kl_loss_coef=0.01),
                                                       optim=OptimizerConfig(lr=1e-5)), with_reference=True)
    g = torch.Generator().manual_seed(0)
    toks = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (12, 9, 14, 10)]
    batch = {"tokens": toks, "response_lengths": [5, 4, 6, 3], "rewards": [1.0, 0.0, 0.3, 0.9], "loss_masks": [[1] * r for r in (5, 4, 6, 3)],
             "group_index": [0, 0, 1, 1]}
    m = actor.train(0, batch)
    assert [len(e) for e in batch["entropy"]] == [5, 4, 6, 3] and [len(e) for e in batch["ref_entropy"]] == [5, 4, 6, 3]
    assert all(float(e.min()) >= 0 for e in batch["entropy"])
    assert m["rollout/entropy"] > 0 and abs(m["rollout/entropy"] - m["rollout/ref_entropy"]) < 1e-5      # reference == initial policy
