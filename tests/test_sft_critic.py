"""SFT data + trainer path, critic (value) training, perplexity eval (CPU, tiny model)."""
import json
import math

import torch

from relax_b200.algo.loss import LossConfig
from relax_b200.data.sft import StreamingSFTDataset, pack_batches, render_chat, to_train_sample
from relax_b200.models.config import get_config
from relax_b200.train.actor import TrainActor, TrainConfig
from relax_b200.train.optimizer import OptimizerConfig


def _tok(s):
    return [3 + (ord(c) % 200) for c in s]


def test_render_chat_masks_assistant_only():
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}, {"role": "user", "content": "k"},
            {"role": "assistant", "content": "bye"}]
    toks, mask = render_chat(msgs, _tok, eos=2)
    assert len(toks) == len(mask) and toks.count(2) == 2
    s = to_train_sample(toks, mask)
    assert s["response_length"] == len(s["loss_mask"]) and sum(s["loss_mask"]) == sum(mask)
    assert s["loss_mask"][0] == 1 and to_train_sample(_tok("abc"), [0, 0, 0]) is None


def test_streaming_dataset_shards_and_resumes(tmp_path):
    files = []
    for i in range(2):
        p = tmp_path / f"s{i}.jsonl"
        with open(p, "w") as f:
            for j in range(5):
                f.write(json.dumps({"prompt": f"q{i}{j}", "response": f"answer {i}{j}"}) + "\n")
        files.append(str(p))
    all_ = list(StreamingSFTDataset(files, _tok))
    assert len(all_) == 10
    r0 = list(StreamingSFTDataset(files, _tok, dp_rank=0, dp_size=2))
    r1 = list(StreamingSFTDataset(files, _tok, dp_rank=1, dp_size=2))
    assert len(r0) == len(r1) == 5 and [s["tokens"] for s in r0] == [s["tokens"] for s in all_[0::2]]
    ds = StreamingSFTDataset(files, _tok)
    it = iter(ds)
    first = [next(it) for _ in range(7)]
    st = ds.state_dict()
    ds2 = StreamingSFTDataset(files, _tok)
    ds2.load_state_dict(st)
    rest = list(ds2)
    assert [s["tokens"] for s in first + rest] == [s["tokens"] for s in all_]
    batches = list(pack_batches(all_, max_tokens=3 * len(all_[0]["tokens"])))
    assert sum(len(b["tokens"]) for b in batches) == 10 and all(len(b["tokens"]) <= 3 for b in batches)


def _cfg(role_lr=2e-3):
    return TrainConfig(global_batch_size=4, max_tokens_per_gpu=256, pad_multiple=1,
                       loss=LossConfig(), optim=OptimizerConfig(lr=role_lr, clip_grad=1.0, weight_decay=0.0))


def test_sft_training_reduces_nll():
    torch.manual_seed(0)
    actor = TrainActor(get_config("tiny"), _cfg(), role="sft")
    samples = [to_train_sample(*render_chat([{"role": "user", "content": "ab"}, {"role": "assistant", "content": "cdcdcd"}], _tok))
               for _ in range(4)]
    batch = {"tokens": [s["tokens"] for s in samples], "response_lengths": [s["response_length"] for s in samples],
             "loss_masks": [s["loss_mask"] for s in samples]}
    before = actor.evaluate_ppl(batch)["eval/nll"]
    for _ in range(8):
        m = actor.train_sft(batch)
    after = actor.evaluate_ppl(batch)
    assert after["eval/nll"] < before - 0.5 and math.isfinite(m["grad_norm"])
    assert abs(after["eval/ppl"] - math.exp(after["eval/nll"])) < 1e-6


def test_critic_fits_returns():
    torch.manual_seed(0)
    cfg = get_config("tiny", value_head=True)
    actor = TrainActor(cfg, _cfg(5e-3), role="critic")
    toks = [[5, 6, 7, 8, 9, 10], [11, 12, 13, 14]]
    rl = [3, 2]
    batch = {"tokens": toks, "response_lengths": rl, "loss_masks": [[1.0] * r for r in rl]}
    v0 = actor.compute_values(batch)["values"]
    assert [len(v) for v in v0] == rl
    batch["values"] = [v.clone() for v in v0]
    batch["returns"] = [torch.full((r,), 1.0) for r in rl]
    err0 = sum(float(((v - 1.0) ** 2).sum()) for v in v0)
    for _ in range(10):
        m = actor.train_critic(0, batch)
    v1 = actor.compute_values(batch)["values"]
    err1 = sum(float(((v - 1.0) ** 2).sum()) for v in v1)
    assert err1 < 0.5 * err0 and "value_loss" in m


def test_freeze_and_only_train_lists():
    import pytest
    from relax_b200.config.arguments import parse_args, train_config_from_args

    a = parse_args(["--model-name", "tiny", "--colocate", "--only-train-params-name-list", r"layers\.1\.", "--freeze-params-name-list", "layer_norm"])
    tc = train_config_from_args(a)
    tc.global_batch_size, tc.pad_multiple, tc.max_tokens_per_gpu = 4, 1, 256
    actor = TrainActor(get_config("tiny"), tc, role="sft")
    names = [n for n, p in actor.model.named_parameters() if p.requires_grad]
    assert names and all(".layers.1." in n and "layer_norm" not in n for n in names)
    before = {n: p.detach().clone() for n, p in actor.model.named_parameters()}
    samples = [to_train_sample(*render_chat([{"role": "user", "content": "ab"}, {"role": "assistant", "content": "cdcd"}], _tok)) for _ in range(4)]
    actor.train_sft({"tokens": [s["tokens"] for s in samples], "response_lengths": [s["response_length"] for s in samples],
                     "loss_masks": [s["loss_mask"] for s in samples]})
    changed = {n for n, p in actor.model.named_parameters() if not torch.equal(p, before[n])}
    assert changed and changed <= set(names)
    with pytest.raises(ValueError):
        TrainActor(get_config("tiny"), _cfg().__class__(only_train_params_name_list=["nothing_matches"]), role="sft")


def test_ppo_with_critic_in_the_colocated_loop():
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO

    cfg = ColocateConfig(model=get_config("tiny"),
                         train=TrainConfig(advantage_estimator="ppo", global_batch_size=4, n_samples_per_prompt=2, pad_multiple=1,
                                           max_tokens_per_gpu=256, gamma=1.0, lambd=0.95, loss=LossConfig(),
                                           optim=OptimizerConfig(lr=1e-4)),
                         rollout_batch_size=2, prompt_len=8, max_response_len=8, kv_blocks=64, num_prompts=16,
                         rm_type="token_sum_parity", critic_lr=5e-3)
    run = ColocatedGRPO(cfg)
    assert run.critic is not None and run.critic.role == "critic" and run.critic.cfg.optim.lr == 5e-3
    w0 = run.critic.model.value_head.weight.detach().clone()
    m = run.step()
    assert "critic/loss" in m or any(k.startswith("critic/") for k in m)
    assert not torch.equal(run.critic.model.value_head.weight.detach(), w0)      # the critic was updated
    assert math.isfinite(m["grad_norm"])


def test_critic_only_warmup_steps_leave_the_policy_untouched():
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO

    cfg = ColocateConfig(model=get_config("tiny"),
                         train=TrainConfig(advantage_estimator="ppo", global_batch_size=4, n_samples_per_prompt=2, pad_multiple=1,
                                           max_tokens_per_gpu=256, loss=LossConfig(), optim=OptimizerConfig(lr=1e-2)),
                         rollout_batch_size=2, prompt_len=8, max_response_len=8, kv_blocks=64, num_prompts=16,
                         rm_type="token_sum_parity", critic_lr=5e-3, num_critic_only_steps=1)
    run = ColocatedGRPO(cfg)
    p0 = run.actor.param_buf.clone()
    c0 = run.critic.param_buf.clone()
    run.step()
    assert torch.equal(run.actor.param_buf, p0) and not torch.equal(run.critic.param_buf, c0)
    run.step()
    assert not torch.equal(run.actor.param_buf, p0)


def test_ppo_resume_restores_the_critic(tmp_path):
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    common = ["--model-name", "tiny", "--colocate", "--advantage-estimator", "ppo", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2",
              "--global-batch-size", "4", "--rollout-max-response-len", "8", "--rm-type", "token_sum_parity", "--critic-lr", "5e-3",
              "--save", str(tmp_path / "ck"), "--load", str(tmp_path / "ck"), "--save-interval", "1"]
    c = Controller(parse_args(common + ["--num-rollout", "1"]), device="cpu")
    c.training_loop()
    trained = c.runner.critic.param_buf.clone()
    assert (tmp_path / "ck_critic").is_dir()
    c2 = Controller(parse_args(common + ["--num-rollout", "2"]), device="cpu")
    assert torch.equal(c2.runner.critic.param_buf, trained) and c2.start_rollout_id == 1
