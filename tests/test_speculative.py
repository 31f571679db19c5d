"""Speculative decoding in the rollout engine (draft = the model's MTP block): greedy outputs equal plain decoding
whether proposals are rejected or accepted, the weights of the block arrive through the sync plan, prompt sharing
and stop conditions behave, and the statistics count."""
import pytest
import torch

from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel
from relax_b200.parallel.state import single_process_state
from relax_b200.rollout.engine import RolloutEngine, SamplingParams
from relax_b200.weight_sync.plan import TrainerLayout, build_plan
from relax_b200.weight_sync.sync import WeightSync


def _engines(seed=5, **kw):
    cfg = get_config("tiny", mtp_num_layers=1)
    model = GPTModel(cfg, single_process_state(), seed=seed)
    params = {k: v.detach() for k, v in model.named_parameters()}
    plain = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=256, block_size=8, **kw)
    spec = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=256, block_size=8, speculative=True, **kw)
    WeightSync(cfg, TrainerLayout(tp=1), 1, [0], [0]).update_weights(params, plain.weights, plain, version=1)
    WeightSync(cfg, TrainerLayout(tp=1), 1, [0], [0], plan=build_plan(cfg, TrainerLayout(tp=1), 1, mtp=True)) \
        .update_weights(params, spec.weights, spec, version=1)
    return cfg, model, plain, spec


def test_layout_and_plan_carry_the_mtp_block():
    cfg, model, plain, spec = _engines()
    L = cfg.num_layers
    assert spec.kv.shape[0] == L + 1 and plain.kv.shape[0] == L
    # the policy's own tensors sit at the same offsets with and without the block
    assert all(spec.weights.offsets[k] == plain.weights.offsets[k] for k in plain.weights.offsets)
    p = dict(model.named_parameters())
    assert torch.equal(spec.weights.p["mtp.eh_proj"], p["mtp.layers.0.eh_proj.weight"])
    assert torch.equal(spec.weights.p["mtp.final_norm"], p["mtp.layers.0.final_layernorm.weight"])
    assert torch.equal(spec.weights.p[f"layers.{L}.o"], p["mtp.layers.0.transformer_layer.self_attention.linear_proj.weight"])
    assert torch.equal(spec.weights.p[f"layers.{L}.down"], p["mtp.layers.0.transformer_layer.mlp.linear_fc2.weight"])
    with pytest.raises(ValueError, match="multi-token-prediction"):
        RolloutEngine(get_config("tiny"), device="cpu", dtype=torch.float32, speculative=True)


def test_greedy_output_is_unchanged_with_rejected_and_with_accepted_proposals():
    cfg, model, plain, spec = _engines()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 9, 16, 23)]
    prompts.append(list(prompts[1]))                      # same prompt and group key as request 1: a follower
    keys = [0, 1, 2, 3, 1]
    sp = SamplingParams(temperature=0.0, max_new_tokens=12)
    want = plain.generate(prompts, sp, group_keys=keys)
    got = spec.generate(prompts, sp, group_keys=keys)
    for a, b in zip(want, got):
        assert a.output == b.output
        assert torch.allclose(torch.tensor(a.logprobs), torch.tensor(b.logprobs), atol=1e-5)
    assert spec.stats["spec_draft_tokens"] > 0 and got[0].spec_verify > 0
    # an untrained block proposes badly: force every proposal to be the token plain decoding will pick, so that every
    # verify pass takes the two-token path (second row valid, draft block run on two positions)
    truth = {tuple(r.prompt): r.output for r in want}
    real = spec._decode_speculative

    def oracle_drafts():
        for r in spec.running:
            out = truth[tuple(r.prompt)]
            r._draft = out[len(r.output):len(r.output) + spec.speculative_steps] or None
        real()

    spec._decode_speculative = oracle_drafts
    before = spec.stats.get("spec_accepted_tokens", 0)
    again = spec.generate(prompts, sp, group_keys=keys)
    for a, b in zip(want, again):
        assert a.output == b.output
        assert torch.allclose(torch.tensor(a.logprobs), torch.tensor(b.logprobs), atol=1e-5)
        assert b.spec_accept == b.spec_draft >= 5 and b.spec_verify <= 7     # 11 tokens after the prefill's in about 6 passes
    assert spec.stats["spec_accepted_tokens"] - before == sum(r.spec_accept for r in again)


def test_chained_proposals_three_per_pass():
    """``speculative_steps = 3``: four rows per verify pass; with proposals that plain decoding confirms, four tokens
    per pass; with the untrained block's own (chained) proposals the output is still plain decoding's."""
    cfg, model, plain, spec = _engines()
    spec.speculative_steps = 3
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (6, 13, 21)]
    prompts.append(list(prompts[0]))
    keys = [0, 1, 2, 0]
    sp = SamplingParams(temperature=0.0, max_new_tokens=14)
    want = plain.generate(prompts, sp, group_keys=keys)
    got = spec.generate(prompts, sp, group_keys=keys)
    assert [r.output for r in got] == [r.output for r in want]
    assert all(r.spec_draft > r.spec_verify for r in got)                # more than one proposal per pass was checked
    truth = {tuple(r.prompt): r.output for r in want}
    real = spec._decode_speculative

    def oracle_drafts():
        for r in spec.running:
            out = truth[tuple(r.prompt)]
            r._draft = out[len(r.output):len(r.output) + 3] or None
        real()

    spec._decode_speculative = oracle_drafts
    again = spec.generate(prompts, sp, group_keys=keys)
    for a, b in zip(want, again):
        assert a.output == b.output and torch.allclose(torch.tensor(a.logprobs), torch.tensor(b.logprobs), atol=1e-5)
        assert b.spec_accept == b.spec_draft and b.spec_verify == 4      # 13 tokens after the prefill's: 4 + 4 + 4 + 1
    # sampling stays well-formed
    del spec._decode_speculative
    c = spec.generate(prompts, SamplingParams(temperature=1.0, max_new_tokens=11), group_keys=keys)
    assert all(len(r.output) == len(r.logprobs) == 11 for r in c)


def test_the_engine_drafts_what_the_trainers_block_predicts():
    """The proposal after a prefill and after decode steps is the arg-max of the trainer-side MTP block on the same
    tokens (full recomputation with the training code), i.e. the block's paged cache is kept right."""
    cfg, model, plain, spec = _engines(seed=9)
    from relax_b200.models.mtp import shift_in_sequence

    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(3, cfg.vocab_size, (11,), generator=g).tolist()
    spec.add_request(prompt, SamplingParams(temperature=0.0, max_new_tokens=8))

    def trainer_draft(seq):
        t = torch.tensor(seq)
        pos = torch.arange(len(seq))
        cu = torch.tensor([0, len(seq)], dtype=torch.int32)
        with torch.no_grad():
            _, pre = model(t, pos, cu, max_seqlen=len(seq), return_prenorm=True)
            tok1, _ = shift_in_sequence(t, cu, 1)
            cos, sin = model.rope_tables(pos)
            emb = model.embedding.word_embeddings(tok1, False)
            _, hn = model.mtp.layers[0](pre, emb, cos, sin, cu, len(seq))
            logits = hn.float() @ model.lm_head_weight()[:cfg.vocab_size].float().t()
        return int(logits[len(seq) - 2].argmax())        # row n-2 holds (h_{n-2}, token n-1) and predicts token n

    for _ in range(5):
        spec.step()
        r = spec.running[0]
        assert r._draft == [trainer_draft(r.prompt + r.output)], len(r.output)


def test_stop_token_and_length_limits_under_speculation():
    cfg, model, plain, spec = _engines()
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(3, cfg.vocab_size, (7,), generator=g).tolist()
    ref = plain.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=10))[0]
    stop = ref.output[4]
    a = plain.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=10, stop_token_ids=(stop,)))[0]
    b = spec.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=10, stop_token_ids=(stop,)))[0]
    assert a.output == b.output and b.finish_reason == "stop" and b.output[-1] == stop
    for n in (1, 2, 3):
        b = spec.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=n))[0]
        assert b.output == ref.output[:n] and b.finish_reason == "length"
    # sampling with temperature: lengths and log-probs are those of a policy sample (finite, one per token)
    c = spec.generate([prompt] * 3, SamplingParams(temperature=1.0, top_p=0.9, max_new_tokens=9), group_keys=[0, 0, 0])
    assert all(len(r.output) == len(r.logprobs) == 9 and all(x <= 0 for x in r.logprobs) for r in c)
    assert spec.bm.num_free == spec.bm.num_blocks - (1 if spec._scratch_block else 0) or spec.bm.num_free > 0


def test_speculative_rollouts_in_the_colocated_loop():
    """``--sglang-speculative-algorithm EAGLE`` with an MTP-trained policy: rollouts are drafted by the MTP block, the
    block's weights follow the trainer through the sync plan, and training (policy + MTP loss) goes on as usual."""
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    with pytest.raises(ValueError, match="mtp-num-layers"):
        parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--sglang-speculative-algorithm", "EAGLE"])
    with pytest.warns(UserWarning, match="rows per request"):
        a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2",
                        "--global-batch-size", "8", "--num-rollout", "2", "--rollout-max-response-len", "8", "--lr", "1e-2",
                        "--rm-type", "token_sum_parity", "--mtp-num-layers", "1", "--enable-mtp-training",
                        "--sglang-speculative-algorithm", "EAGLE", "--sglang-speculative-num-steps", "2",
                        "--sglang-speculative-eagle-topk", "1", "--sglang-speculative-num-draft-tokens", "4"])
    c = Controller(a, device="cpu")
    run = c.runner
    assert run.engine.speculative and run.engine.speculative_steps == 2 and run.engine.kv.shape[0] == run.cfg.model.num_layers + 1
    m = run.step()
    assert m["rollout/spec_draft_tokens"] > 0 and 0.0 <= m["rollout/spec_accept_rate"] <= 1.0 and "mtp_loss" in m
    # rollout log-probs are the policy's: the trainer reproduces them on the sampled tokens
    assert m["train_rollout_logprob_abs_diff"] < 1e-4
    p = dict(run.actor.named_local_params())
    L = run.cfg.model.num_layers
    assert torch.equal(run.engine.weights.p["mtp.eh_proj"], p["mtp.layers.0.eh_proj.weight"].detach().to(run.engine.weights.p["mtp.eh_proj"].dtype))
    assert torch.equal(run.engine.weights.p[f"layers.{L}.down"],
                       p["mtp.layers.0.transformer_layer.mlp.linear_fc2.weight"].detach().to(run.engine.weights.p[f"layers.{L}.down"].dtype))
    run.step()
    run.close()


def test_a_trained_block_halves_the_number_of_passes():
    """Policy and MTP block trained (SFT with the MTP loss) on a predictable sequence: the block's proposals are
    accepted and 24 tokens take 12 verify passes instead of 23 decode passes."""
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    torch.manual_seed(0)
    cfg = get_config("tiny", mtp_num_layers=1)
    actor = TrainActor(cfg, TrainConfig(global_batch_size=16, enable_mtp_training=True, mtp_loss_scaling_factor=1.0, pad_multiple=1,
                                        max_tokens_per_gpu=4096, optim=OptimizerConfig(lr=3e-3)), role="sft")

    def seq(start, n):
        return [3 + (start + 5 * i) % 40 for i in range(n)]

    batch = {"tokens": [seq(s, 40) for s in range(16)], "response_lengths": [39] * 16, "total_lengths": [40] * 16,
             "loss_masks": [[1] * 39 for _ in range(16)]}
    for _ in range(30):
        m = actor.train_sft(batch)
    assert m["loss"] < 0.01 and m["mtp_loss"] < 0.01
    spec = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=256, block_size=8, speculative=True)
    WeightSync(cfg, TrainerLayout(tp=1), 1, [0], [0], plan=build_plan(cfg, TrainerLayout(tp=1), 1, mtp=True)) \
        .update_weights(dict(actor.named_local_params()), spec.weights, spec, version=1)
    out = spec.generate([seq(s, 8) for s in (1, 7, 20)], SamplingParams(temperature=0.0, max_new_tokens=24))
    for s, r in zip((1, 7, 20), out):
        assert r.output == seq(s, 32)[8:]
        assert r.spec_accept == r.spec_draft == 11 and r.spec_verify == 12
    assert spec.stats["steps"] == 13 and spec.stats["spec_accepted_tokens"] == 33
    # three chained proposals per pass (the block runs on its own output for the second and third): 6 passes
    spec.speculative_steps = 3
    out = spec.generate([seq(s, 8) for s in (1, 7, 20)], SamplingParams(temperature=0.0, max_new_tokens=24))
    assert all(r.output == seq(s, 32)[8:] and r.spec_verify == 6 and r.spec_accept == 17 for s, r in zip((1, 7, 20), out))


def test_hf_checkpoint_with_mtp_block_loads_into_a_speculating_engine(tmp_path):
    """A Hugging Face checkpoint of an MTP model fills a speculating engine directly (serving without a trainer): the
    draft block's tensors arrive with the rest and the engine's output equals a plain engine's."""
    from relax_b200.checkpoint import hf as H

    cfg, model, plain, spec = _engines(seed=21)
    d = str(tmp_path / "hf")
    H.save_hf_checkpoint(d, cfg, H.convert_state_to_hf(cfg, {k: v.detach() for k, v in model.named_parameters()}))
    fresh = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8, speculative=True, speculative_steps=2)
    fresh.weights.flat.zero_()
    H.load_hf_into_rollout(d, cfg, fresh.weights)
    for k, v in spec.weights.p.items():
        assert torch.equal(fresh.weights.p[k], v), k
    prompt = [5, 9, 17, 33, 2, 8]
    sp = SamplingParams(temperature=0.0, max_new_tokens=9)
    assert fresh.generate([prompt], sp)[0].output == plain.generate([prompt], sp)[0].output
