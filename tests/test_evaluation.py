"""Evaluation rollouts: pass@k, per-set metrics, dataset loading, the hook in the colocated loop (CPU)."""
import json
import math

import pytest
import torch

from relax_b200.rollout import evaluation as E
from relax_b200.types import Sample, SampleStatus


def test_pass_at_k_estimator():
    assert E.pass_at_k(4, 0, 2) == 0.0 and E.pass_at_k(4, 4, 1) == 1.0 and E.pass_at_k(4, 3, 2) == 1.0
    assert abs(E.pass_at_k(4, 1, 1) - 0.25) < 1e-12
    assert abs(E.pass_at_k(4, 1, 2) - (1 - math.comb(3, 2) / math.comb(4, 2))) < 1e-12
    with pytest.raises(ValueError):
        E.pass_at_k(2, 1, 3)


def test_summary_metrics():
    def S(r, n, trunc=False):
        return Sample(reward=r, response_length=n, status=SampleStatus.TRUNCATED if trunc else SampleStatus.COMPLETED)
    groups = [[S(1.0, 10), S(0.0, 20), S(0.0, 30, True), S({"score": 1.0}, 40)], [S(0.0, 5), S(0.0, 5), S(0.0, 5), S(0.0, 5)]]
    m = E.summarize("aime", groups)
    assert m["eval/aime"] == 0.25 and m["eval/aime-truncated_ratio"] == 0.125 and m["eval/aime/response_len/max"] == 40
    assert abs(m["eval/aime-pass@1"] - 0.25) < 1e-12 and m["eval/aime-pass@4"] == 0.5 and "eval/aime-pass@8" not in m
    assert abs(m["eval/aime-pass@2"] - (1 - math.comb(2, 2) / math.comb(4, 2)) / 2) < 1e-12


def test_load_sets_with_overrides(tmp_path):
    f = tmp_path / "a.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": "x" * n, "label": n}) for n in (3, 50, 5, 7)) + "\n")
    sets = E.load_eval_datasets(["a", str(f)], lambda s: [ord(c) for c in s], n_samples_per_prompt=2, max_prompt_len=10, size=2,
                                overrides={"a": {"temperature": 0.6, "max_response_len": 9}})
    assert len(sets) == 1 and sets[0].labels == [3, 5] and sets[0].temperature == 0.6 and sets[0].n_samples_per_prompt == 2
    with pytest.raises(ValueError):
        E.load_eval_datasets(["a"], len)
    with pytest.raises(KeyError):
        E.load_eval_datasets(["a", str(f)], lambda s: [1], overrides={"a": {"nope": 1}})


def test_colocated_loop_runs_eval_on_schedule():
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    g = torch.Generator().manual_seed(0)
    ds = E.EvalDataset("held", [torch.randint(3, 1000, (8,), generator=g).tolist() for _ in range(3)], n_samples_per_prompt=2,
                       temperature=1.0, max_response_len=6)
    cfg = ColocateConfig(model=get_config("tiny"), train=TrainConfig(global_batch_size=4, n_samples_per_prompt=2, pad_multiple=1,
                         max_tokens_per_gpu=256, loss=LossConfig(), optim=OptimizerConfig(lr=1e-4)),
                         rollout_batch_size=2, prompt_len=8, max_response_len=8, kv_blocks=64, num_prompts=16,
                         eval_datasets=[ds], eval_interval=2)
    run = ColocatedGRPO(cfg)
    m0, m1, m2 = run.step(), run.step(), run.step()
    assert "eval/held" in m0 and "eval/held-pass@2" in m0 and m0["eval/held/num_prompts"] == 3.0
    assert "eval/held" not in m1 and "eval/held" in m2
    assert m0["eval/held/response_len/max"] <= 6


def test_entrypoint_flags_reach_the_loop(tmp_path):
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    f = tmp_path / "held.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": f"question {i}", "label": i}) for i in range(3)) + "\n")
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2",
                    "--global-batch-size", "4", "--num-rollout", "1", "--rollout-max-response-len", "8",
                    "--eval-interval", "1", "--eval-prompt-data", "held", str(f), "--n-samples-per-eval-prompt", "2",
                    "--eval-max-response-len", "4"])
    c = Controller(a, device="cpu")
    runner = c.runner if hasattr(c, "runner") else c.build_runner()
    m = runner.step()
    assert m["eval/held/num_prompts"] == 3.0 and "eval/held-pass@2" in m and m["eval/held/response_len/max"] <= 4


def test_dump_replay_passrate_epochs_and_reference_refresh(tmp_path):
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    f = tmp_path / "train.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": f"q{i}", "label": str(i)}) for i in range(4)) + "\n")
    common = ["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
              "--rollout-max-response-len", "8", "--rm-type", "token_sum_parity", "--prompt-data", str(f), "--input-key", "prompt",
              "--label-key", "label"]
    dumps, train = tmp_path / "dumps", tmp_path / "train_data"
    a = parse_args(common + ["--num-epoch", "1", "--save-debug-rollout-data", str(dumps), "--save-debug-train-data", str(train),
                             "--log-passrate", "--use-kl-loss", "--kl-loss-coef", "0.01", "--ref-update-interval", "2"])
    c = Controller(a, device="cpu")
    hist = c.training_loop()
    assert len(hist) == 2 and a.num_rollout == 2                       # 4 prompts / 2 per rollout, one epoch
    assert "rollout/pass-pass@1" in hist[0] and "rollout/pass-pass@2" in hist[0]
    assert "ref_updated" not in hist[0] and hist[1].get("ref_updated") == 1.0
    assert sorted(p.name for p in dumps.iterdir()) == ["rollout_0.jsonl", "rollout_1.jsonl"]
    saved = torch.load(train / "train_0_rank0.pt")
    assert len(saved["tokens"]) == 4 and "rewards" in saved
    # replay the dumped rollouts through the trainer: same rewards, no generation
    b = parse_args(common + ["--num-rollout", "1", "--load-debug-rollout-data", str(dumps)])
    c2 = Controller(b, device="cpu")
    calls = []
    c2.runner.engine.generate = lambda *x, **k: calls.append(1)
    m = c2.runner.step()
    assert not calls and abs(m["raw_reward_mean"] - hist[0]["raw_reward_mean"]) < 1e-9


def test_reward_key_selects_the_dict_entry():
    def S(r):
        return Sample(reward=r, response_length=1, status=SampleStatus.COMPLETED)
    groups = [[S({"score": 0.0, "acc": 1.0}), S({"score": 0.0, "acc": 0.0})]]
    assert E.summarize("x", groups)["eval/x"] == 0.0
    m = E.summarize("x", groups, reward_key="acc")
    assert m["eval/x"] == 0.5 and m["eval/x-pass@2"] == 1.0
