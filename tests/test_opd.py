"""On-policy distillation divergences against brute-force statements."""
import math

import pytest
import torch

from relax_b200.algo import opd


def _dists(R=5, V=11, seed=0):
    g = torch.Generator().manual_seed(seed)
    s = torch.log_softmax(torch.randn(R, V, generator=g), -1)
    t = torch.log_softmax(torch.randn(R, V, generator=g) * 1.5, -1)
    return s, t


def test_sampled_token_estimators():
    s, t = _dists()
    ids = torch.tensor([0, 3, 5, 7, 10])
    sl, tl = s[torch.arange(5), ids], t[torch.arange(5), ids]
    assert torch.allclose(opd.token_kl(sl, tl, "reverse_kl"), sl - tl)
    r = sl - tl
    assert torch.allclose(opd.token_kl(sl, tl, "low_var_kl"), torch.exp(-r) - 1 + r)
    with pytest.raises(ValueError):
        opd.token_kl(sl, tl, "jsd")
    c = opd.token_kl(torch.tensor([-50.0]), torch.tensor([-1.0]), "reverse_kl", log_prob_min_clamp=-10.0)
    assert float(c) == -9.0


def test_full_support_topk_equals_exact_divergences():
    s, t = _dists()
    rev = (s.exp() * (s - t)).sum(-1)
    fwd = (t.exp() * (t - s)).sum(-1)
    for mode in ("tail", "norm", "trunc"):
        assert torch.allclose(opd.token_kl(s, t, "reverse_kl", norm_mode=mode), rev, atol=1e-5)
        assert torch.allclose(opd.token_kl(s, t, "forward_kl", norm_mode=mode), fwd, atol=1e-5)
    a = 0.3
    m = torch.log((1 - a) * s.exp() + a * t.exp())
    jsd = (1 - a) * (s.exp() * (s - m)).sum(-1) + a * (t.exp() * (t - m)).sum(-1)
    assert torch.allclose(opd.token_kl(s, t, "jsd", alpha=a, norm_mode="trunc"), jsd, atol=1e-5)


def test_tail_bin_and_union_mask():
    s, t = _dists(V=16)
    ids_s, ids_t = s.topk(4, -1).indices, t.topk(4, -1).indices
    ids, lens = opd.union_ids(ids_s, ids_t)
    assert ids.shape[0] == 5 and int(lens.min()) >= 4 and int(lens.max()) <= 8
    for r in range(5):
        assert set(ids[r, :lens[r]].tolist()) == set(ids_s[r].tolist()) | set(ids_t[r].tolist())
    sk, tk = s.gather(-1, ids), t.gather(-1, ids)
    got = opd.per_token_signal("union", student_topk_lp=sk, teacher_topk_lp=tk, k_lengths=lens, kl_type="reverse_kl",
                               norm_mode="tail")
    for r in range(5):
        k = int(lens[r])
        ps, pt = sk[r, :k].exp(), tk[r, :k].exp()
        want = (ps * (sk[r, :k] - tk[r, :k])).sum() + (1 - ps.sum()) * (torch.log(1 - ps.sum()) - torch.log(1 - pt.sum()))
        assert abs(float(got[r]) - float(want)) < 1e-5
        assert float(got[r]) >= -1e-6   # a KL between two proper distributions (K ids + tail)


def test_advantage_shaping_and_loss():
    adv = [torch.zeros(3), torch.ones(2)]
    sig = [torch.tensor([0.5, 3.0, -1.0]), torch.tensor([0.1, 0.2])]
    out = opd.apply_to_advantages(adv, sig, coef=2.0, per_token_clip=1.0)
    assert torch.allclose(out[0], torch.tensor([-1.0, -2.0, 2.0])) and torch.allclose(out[1], torch.tensor([0.8, 0.6]))
    assert opd.apply_to_advantages(adv, sig, coef=0.0) is adv
    x = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0], requires_grad=True)
    loss = opd.opd_loss(x, [torch.tensor([1.0, 0.0, 1.0]), torch.tensor([1.0, 1.0])], [3, 2], coef=0.5)
    assert abs(float(loss) - 0.5 * (1 + 3 + 4 + 5) / 4) < 1e-6
    loss.backward()
    assert torch.allclose(x.grad, torch.tensor([0.125, 0.0, 0.125, 0.125, 0.125]))


def test_teacher_pool_splits_work_and_fails_over():
    import pytest
    from relax_b200.algo.opd import TeacherPool

    class T:
        def __init__(self, tag, fail=False):
            self.tag, self.fail, self.calls = tag, fail, 0

        def score(self, batch):
            self.calls += 1
            if self.fail:
                raise RuntimeError("engine died")
            return [torch.full((len(t),), float(self.tag)) for t in batch["tokens"]]

    batch = {"tokens": [[1] * (i + 1) for i in range(7)], "response_lengths": [1] * 7, "temperature": 1.0}
    a, b = T(1), T(2)
    out = TeacherPool([a, b]).score(batch)
    assert [len(o) for o in out] == list(range(1, 8)) and a.calls == 1 and b.calls == 1
    assert {float(o[0]) for o in out} == {1.0, 2.0}
    bad = T(9, fail=True)
    pool = TeacherPool([bad, T(3)], retry_after_s=1000)
    out = pool.score(batch)
    assert all(float(o[0]) == 3.0 for o in out) and pool.failures == 1 and pool.healthy() == [1]
    pool.score(batch)
    assert bad.calls == 1                      # not retried before retry_after_s
    pool.retry_after_s = 0.0
    assert pool.healthy() == [0, 1]
    with pytest.raises(RuntimeError):
        TeacherPool([T(1, fail=True)]).score(batch)


def test_opd_penalty_in_the_trainer_pulls_towards_the_teacher(tmp_path):
    from relax_b200.algo.loss import LossConfig
    from relax_b200.checkpoint import hf as H
    from relax_b200.config.arguments import parse_args
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.orchestration.controller import Controller

    cfg = get_config("tiny")
    teacher = GPTModel(cfg, seed=77)
    d = str(tmp_path / "teacher")
    H.save_hf_checkpoint(d, cfg, H.convert_state_to_hf(cfg, {k: v.detach() for k, v in teacher.named_parameters()}))
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "8", "--opd-type", "megatron", "--opd-teacher-load", d,
                    "--opd-kl-coef", "0.5", "--lr", "1e-4"])
    c = Controller(a, device="cpu")
    actor = c.runner.actor
    assert "teacher" in actor.snapshots and actor.cfg.opd_kl_coef == 0.5
    # the policy itself was not replaced by the teacher
    own = GPTModel(cfg, seed=a.seed)
    name = "decoder.layers.0.mlp.linear_fc2.weight"
    assert torch.equal(dict(actor.model.named_parameters())[name].detach(), dict(own.named_parameters())[name].detach())
    assert actor._active_tag == "actor"
    m = c.runner.step()
    assert "opd_kl" in m and m["opd_kl"] != 0.0 and math.isfinite(m["grad_norm"])


def test_remote_teacher_over_http_and_pool_failover():
    """``--opd-teacher-urls``: a teacher served over HTTP scores the batch; a dead URL in the pool is marked
    unhealthy and its slice is re-run on the live one; the colocated loop trains with the remote scores."""
    import torch

    from relax_b200.algo.opd import HTTPTeacher, InProcessTeacher, TeacherPool, serve_teacher
    from relax_b200.models.config import get_config
    from relax_b200.train.actor import TrainActor, TrainConfig

    cfg = get_config("tiny")
    teacher = TrainActor(cfg, TrainConfig(), seed=7, with_optimizer=False)
    srv, _ = serve_teacher(InProcessTeacher(teacher))
    url = f"http://127.0.0.1:{srv.server_address[1]}"
    g = torch.Generator().manual_seed(0)
    batch = {"tokens": [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 14, 11)],
             "response_lengths": [4, 6, 5]}
    ref = teacher.compute_log_prob(batch)["log_probs"]
    got = HTTPTeacher(url).score(batch)
    for a, b in zip(got, ref):
        assert torch.allclose(a, b, atol=1e-6)
    pool = TeacherPool([HTTPTeacher("http://127.0.0.1:9", timeout_s=2.0), HTTPTeacher(url)], timeout_s=5.0)
    got = pool.score(batch)
    assert pool.failures >= 1 and all(torch.allclose(a, b, atol=1e-6) for a, b in zip(got, ref))

    from relax_b200.algo.loss import LossConfig
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO
    from relax_b200.train.optimizer import OptimizerConfig

    run = ColocatedGRPO(ColocateConfig(
        model=cfg, train=TrainConfig(n_samples_per_prompt=2, global_batch_size=8, max_tokens_per_gpu=1024, opd_kl_coef=0.5,
                                     loss=LossConfig(), optim=OptimizerConfig(lr=1e-5)),
        rollout_batch_size=4, prompt_len=8, max_response_len=8, rm_type="parity", opd_teacher_urls=[url]))
    m = run.step()
    assert "opd_reverse_kl" in m or any("opd" in k for k in m), sorted(m)
    run.close()
    srv.shutdown()
    srv.server_close()


def test_topk_log_probs_match_a_plain_softmax_and_drive_the_topk_selections(tmp_path):
    """``compute_topk_log_probs`` against log_softmax of the full logits (fp32), and a training step per top-K token
    selection: teacher = student gives a zero signal, a different teacher a positive one (a KL on the chosen ids)."""
    import torch.nn.functional as F

    from relax_b200.checkpoint import hf as H
    from relax_b200.config.arguments import parse_args
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.orchestration.controller import Controller
    from relax_b200.train.actor import TrainActor, TrainConfig

    cfg = get_config("tiny")
    actor = TrainActor(cfg, TrainConfig(), seed=3, with_optimizer=False)
    g = torch.Generator().manual_seed(0)
    toks = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (13, 9, 17)]
    batch = {"tokens": toks, "response_lengths": [5, 4, 9], "total_lengths": [13, 9, 17]}
    own = actor.compute_topk_log_probs(batch, k=6)
    # reference: full logits of the response positions with plain PyTorch
    w = actor.model.lm_head_weight()[:cfg.vocab_size].float()
    sampled = actor.compute_log_prob(batch)["log_probs"]
    for i, (t, r) in enumerate(zip(toks, batch["response_lengths"])):
        x = torch.tensor(t)
        with torch.no_grad():
            h = actor.model(x, torch.arange(len(t)), torch.tensor([0, len(t)], dtype=torch.int32), max_seqlen=len(t))
        full = F.log_softmax(h[len(t) - r - 1:len(t) - 1].float() @ w.t(), -1)
        val, idx = full.topk(6, -1)
        assert torch.equal(own["ids"][i], idx) and torch.allclose(own["log_probs"][i], val, atol=1e-5)
        # gather mode, with padding, and consistency with the sampled-token pass
        ids = torch.cat([x[len(t) - r:, None], torch.full((r, 1), -1)], -1)
        got = actor.compute_topk_log_probs(batch, ids=[ids if j == i else torch.zeros(batch["response_lengths"][j], 2, dtype=torch.long)
                                                       for j in range(3)])["log_probs"][i]
        assert torch.allclose(got[:, 0], sampled[i].float(), atol=1e-5) and torch.isinf(got[:, 1]).all()

    teacher = GPTModel(cfg, seed=77)
    d = str(tmp_path / "teacher")
    H.save_hf_checkpoint(d, cfg, H.convert_state_to_hf(cfg, {k: v.detach() for k, v in teacher.named_parameters()}))
    base = ["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
            "--num-rollout", "1", "--rollout-max-response-len", "6", "--use-opd", "--opd-teacher-load", d, "--opd-kl-coef", "0.5", "--lr", "1e-4"]
    with pytest.raises(ValueError, match="top-k"):
        parse_args(base + ["--opd-token-selection", "union"])
    with pytest.raises(ValueError, match="both distributions"):
        parse_args(base + ["--opd-kl-type", "jsd"])
    for sel, kl in (("student_topk", "reverse_kl"), ("teacher_topk", "forward_kl"), ("union", "jsd")):
        a = parse_args(base + ["--opd-token-selection", sel, "--opd-log-prob-top-k", "8", "--opd-kl-type", kl])
        assert a.opd_type == "megatron"
        c = Controller(a, device="cpu")
        assert c.runner.actor.cfg.opd_token_selection == sel
        m = c.runner.step()
        assert m["opd_kl"] > 0 and math.isfinite(m["grad_norm"]), (sel, m["opd_kl"])
        c.runner.close()
    a = parse_args(base[:-6] + ["--opd-type", "megatron", "--opd-kl-coef", "0.5", "--opd-topk", "4"])       # short form, no teacher: nothing to distil
    assert a.opd_token_selection == "teacher_topk" and a.opd_log_prob_top_k == 4


def test_loss_mode_and_pure_distillation(tmp_path):
    """``--opd-loss-coef`` (the divergence as a differentiable loss term, with the per-token and importance clips) and
    ``--opd-only-reward`` (the task reward's advantages removed): the loss term equals its definition, and a pure
    distillation step moves the policy towards the teacher."""
    from relax_b200.algo import loss as L
    from relax_b200.algo.ppo_utils import Segments
    from relax_b200.checkpoint import hf as H
    from relax_b200.config.arguments import parse_args
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.orchestration.controller import Controller

    # the term in isolation
    lp = torch.tensor([-1.0, -2.0, -0.5, -3.0], requires_grad=True)
    tlp = torch.tensor([-1.5, -1.0, -0.5, -0.5])
    b = L.LossBatch(seg=Segments.from_lengths([2, 2]), loss_mask=torch.ones(4), advantages=torch.zeros(4),
                    old_log_probs=lp.detach() - 1.0, extras={"teacher_log_probs": tlp})
    cfg = L.LossConfig(opd_loss_coef=2.0, opd_kl_type="reverse_kl", opd_per_token_clip=0.75, opd_is_clip=2.0)
    loss, m = L.policy_loss(lp, torch.zeros(4), b, cfg)
    d = (lp.detach() - tlp).clamp(max=0.75) * 2.0           # ratio e^1 clipped to 2
    assert torch.allclose(m["opd_loss"], d.view(2, 2).mean(1).sum()) and float(m["opd_is_clip_frac"]) == 2.0
    loss.backward()
    # clipped tokens (0.5 -> only token 0 is below the clip... tokens with d > clip pass no gradient)
    raw = lp.detach() - tlp
    assert all((lp.grad[i] == 0) == bool(raw[i] > 0.75) for i in range(4))

    cfgm = get_config("tiny")
    teacher = GPTModel(cfgm, seed=77)
    d_ = str(tmp_path / "teacher")
    H.save_hf_checkpoint(d_, cfgm, H.convert_state_to_hf(cfgm, {k: v.detach() for k, v in teacher.named_parameters()}))
    base = ["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
            "--num-rollout", "3", "--rollout-max-response-len", "6", "--use-opd", "--opd-teacher-load", d_, "--lr", "5e-3"]
    with pytest.raises(ValueError, match="exactly one"):
        parse_args(base + ["--opd-loss-coef", "1.0", "--opd-kl-coef", "0.3"])
    a = parse_args(base + ["--opd-loss-coef", "1.0", "--opd-only-reward", "--opd-per-token-clip", "20"])
    assert a.opd_kl_coef == 0.0
    c = Controller(a, device="cpu")
    assert c.runner.actor.cfg.opd_only_reward and c.runner.actor.cfg.loss.opd_loss_coef == 1.0
    hist = [c.runner.step() for _ in range(3)]
    assert all("opd_loss" in m and math.isfinite(m["grad_norm"]) for m in hist)
    assert all(abs(m["rollout/advantages"]) < 1e-6 for m in hist)         # the task reward does not reach the policy
    assert all(m["pg_loss"] == 0.0 and m["loss"] == pytest.approx(m["opd_loss"], abs=1e-6) for m in hist)   # only the term trains
    c.runner.close()
