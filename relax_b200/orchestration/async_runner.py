"""Builds the fully-async / hybrid pipeline of one process from flags: trainer, rollout engine,
weight sync and the callbacks the role loops need (relax/components/{rollout,actor,actor_fwd,
advantages}.py wired by relax/core/controller.py ``register_all_serve`` :675-763)."""
from __future__ import annotations

import torch

from ..data.convert import convert_samples_to_train_data
from ..parallel.state import GroupInfo, single_process_state
from ..rewards import get_reward_spec
from ..rollout.data_source import RolloutDataSource, SyntheticPromptDataset
from ..rollout.engine import RolloutEngine, SamplingParams
from ..train.actor import TrainActor
from ..types import SampleStatus
from ..weight_sync.plan import TrainerLayout
from ..weight_sync.sync import WeightSync
from .async_pipeline import AsyncPipeline, PipelineConfig
from .controller import _get


class AsyncRunner:
    def __init__(self, pipe: AsyncPipeline, actor: TrainActor, engine: RolloutEngine, timeout: float):
        self.pipe, self.actor, self.engine, self.timeout = pipe, actor, engine, timeout

    def run(self):
        return self.pipe.run(timeout=self.timeout)


class DisaggRunner:
    """Adapter of :class:`~relax_b200.orchestration.disagg.DisaggregatedRL` to the controller's runner protocol."""

    def __init__(self, rl):
        self.rl = rl
        self.actor, self.engine = rl.actor, rl.engine

    def run(self):
        out = self.rl.run()
        if not self.rl.is_trainer:
            return []
        extra = {k: float(v) for k, v in self.rl.stats.items() if isinstance(v, (int, float))}
        return [(rid, {**m, **({f"async/{k}": v for k, v in extra.items()} if rid == out[-1][0] else {})}) for rid, m in out]

    def close(self):
        self.rl.close()


def build_disagg_runner(args, model_cfg, train_cfg, device, start_rollout_id: int = 0) -> DisaggRunner:
    """Trainer and rollout pools on disjoint ranks, placed by ``--resource`` (one process per GPU)."""
    import torch.distributed as dist

    from .disagg import DisaggConfig, DisaggregatedRL
    from .registry import assign_ranks

    world = dist.get_world_size()
    res = dict(getattr(args, "resource_map", None) or {})
    if "actor" not in res or "rollout" not in res:
        n_roll = _get(args, "rollout_num_gpus", None) or world // 2
        res = {"actor": (1, world - n_roll), "rollout": (1, n_roll)}
    ranks = assign_ranks({k: res[k] for k in ("actor", "rollout")}, world, colocate=False)
    plen = _get(args, "rollout_max_prompt_len", 512)
    ctx = _get(args, "rollout_max_context_len", plen + args.rollout_max_response_len)
    page = _get(args, "engine_block_size", 16)
    rtp = _get(args, "rollout_num_gpus_per_engine", 1)
    n_seq = args.rollout_batch_size * args.n_samples_per_prompt // max(1, len(ranks["rollout"]) // rtp)
    cfg = DisaggConfig(
        model=model_cfg, train=train_cfg, trainer_ranks=ranks["actor"], rollout_ranks=ranks["rollout"],
        trainer_tp=args.tensor_model_parallel_size, rollout_tp=rtp, rollout_batch_size=args.rollout_batch_size,
        prompt_len=plen, max_response_len=args.rollout_max_response_len, temperature=args.rollout_temperature,
        top_p=_get(args, "rollout_top_p", 1.0), top_k=_get(args, "rollout_top_k", -1), rm_type=args.rm_type or "parity",
        kv_blocks=_get(args, "kv_blocks", max(64, n_seq * (ctx // page + 2))), kv_block_size=page,
        max_running=_get(args, "engine_max_running", 256), use_cuda_graph=not _get(args, "engine_disable_cuda_graph", False),
        num_rollout=args.num_rollout - start_rollout_id, max_staleness=args.max_staleness,
        update_weights_interval=args.update_weights_interval, seed=args.seed, rollout_seed=args.rollout_seed,
        weight_push=_get(args, "weight_push", "peer"), speculative=bool(_get(args, "engine_speculative_algorithm", None)),
        speculative_steps=int(_get(args, "engine_speculative_num_steps", 1) or 1), num_iters_per_train_update=_get(args, "num_iters_per_train_update", 1) or 1)
    return DisaggRunner(DisaggregatedRL(cfg, device=device))


def build_async_runner(args, model_cfg, train_cfg, device, start_rollout_id: int = 0):
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_world_size() > 1:
        return build_disagg_runner(args, model_cfg, train_cfg, device, start_rollout_id)
    ps = single_process_state()
    need_ref = train_cfg.loss.use_kl_loss or train_cfg.kl_coef != 0
    actor = TrainActor(model_cfg, train_cfg, ps, device=device, seed=args.seed, with_reference=need_ref)
    g = GroupInfo(None, (0,), 0)
    plen = _get(args, "rollout_max_prompt_len", 512)
    ctx = _get(args, "rollout_max_context_len", plen + args.rollout_max_response_len)
    n_seq = args.rollout_batch_size * args.n_samples_per_prompt
    engine = RolloutEngine(model_cfg, g, device=device, dtype=actor.model.dtype,
                           num_kv_blocks=max(64, n_seq * (ctx // 16 + 2)), block_size=16,
                           max_running=_get(args, "sglang_max_running_requests", 256), seed=args.rollout_seed,
                           max_model_len=ctx)
    sync = WeightSync(model_cfg, TrainerLayout(tp=1), 1, [0], [0])
    ds = SyntheticPromptDataset(1 << 14, plen, model_cfg.vocab_size, seed=args.seed)
    source = RolloutDataSource(ds, args.n_samples_per_prompt)
    reward = get_reward_spec(args.rm_type or "parity").fn
    sp = SamplingParams(temperature=args.rollout_temperature, top_p=_get(args, "rollout_top_p", 1.0), top_k=_get(args, "rollout_top_k", -1),
                        max_new_tokens=args.rollout_max_response_len)

    def push(payload):
        params, version = payload
        sync.update_weights(params, engine.weights, engine, version=version)

    push((dict(actor.named_local_params()), actor.weight_version))

    def generate(rid):
        flat = [s for grp in source.get_samples(args.rollout_batch_size) for s in grp]
        res = engine.generate([s.tokens for s in flat], sp, group_keys=[s.group_index for s in flat])
        for s, r in zip(flat, res):
            s.tokens = list(r.prompt) + list(r.output)
            s.response_length = len(r.output)
            s.rollout_log_probs = list(r.logprobs)
            s.weight_versions = sorted(set(r.weight_versions))
            s.status = SampleStatus.TRUNCATED if r.finish_reason == "length" else SampleStatus.COMPLETED
            s.reward = reward(s)
        return flat

    def convert(samples):
        return convert_samples_to_train_data(samples, advantage_estimator=train_cfg.advantage_estimator,
                                             n_samples_per_prompt=train_cfg.n_samples_per_prompt,
                                             rewards_normalization=train_cfg.rewards_normalization,
                                             grpo_std_normalization=train_cfg.grpo_std_normalization)

    def train(rid, batch):
        m = actor.train(rid, batch)
        actor.after_train()
        return m

    def export():
        # a private copy: the trainer keeps stepping while the rollout side applies this version
        return ({k: v.detach().clone() for k, v in actor.named_local_params()}, actor.weight_version)

    cfg = PipelineConfig(num_rollout=args.num_rollout - start_rollout_id, max_staleness=args.max_staleness,
                         rollout_batch_size=args.rollout_batch_size, fully_async=bool(args.fully_async),
                         hybrid=bool(getattr(args, "hybrid", False)), true_on_policy_mode=args.true_on_policy_mode,
                         advantage_estimator=train_cfg.advantage_estimator,
                         update_weights_interval=args.update_weights_interval)
    pipe = AsyncPipeline(cfg, generate_fn=generate, convert_fn=convert, train_fn=train, export_weights_fn=export,
                         push_to_rollout_fn=push, kl_coef=train_cfg.kl_coef, start_rollout_id=start_rollout_id)
    return AsyncRunner(pipe, actor, engine, timeout=float(getattr(args, "async_timeout_s", 3600.0)))
