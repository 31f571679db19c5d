"""Colocated (synchronous, time-shared GPUs) RL loop in SPMD form.

Every process owns one GPU and plays two roles in turn: a rank of a rollout
engine, then a rank of the trainer - the reference's ``--colocate`` mode with
``max_staleness=0`` (one colocated step: relax/components/rollout.py:403-523 +
relax/backends/megatron/actor.py:724-842).  Per step:

1. ``generate``: the rank's engine samples ``n_samples_per_prompt`` responses
   for its share of the prompt batch (group prefix sharing, log-probs returned);
2. rewards + group normalisation; rows are published to the data plane under
   partition ``train_{rollout_id}``;
3. rollout memory is released by tag, trainer state is onloaded;
4. the trainer consumes its rows (task ``actor``): reference / old log-probs,
   advantages, optimizer steps;
5. trainer -> rollout weight sync (block-copy plan), version bump.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..data import transfer_queue as tq
from ..data.convert import convert_samples_to_train_data, custom_meta_rows
from ..models.config import ModelConfig, get_config
from ..parallel.state import GroupInfo, ParallelDims, init_parallel_state, single_process_state
from ..rewards import get_reward_spec
from ..rollout.data_source import RolloutDataSource, SyntheticPromptDataset
from ..rollout.engine import RolloutEngine, SamplingParams
from ..train.actor import TrainActor, TrainConfig
from ..types import Sample, SampleStatus
from ..utils.timer import Timer
from ..weight_sync.plan import TrainerLayout
from ..weight_sync.sync import WeightSync


@dataclass
class ColocateConfig:
    model: ModelConfig = field(default_factory=lambda: get_config("tiny"))
    train: TrainConfig = field(default_factory=TrainConfig)
    trainer_tp: int = 1
    trainer_cp: int = 1
    trainer_pp: int = 1
    trainer_ep: int = 1                  # expert parallelism of the trainer (divides dp x cp; experts keep TP 1)
    rollout_tp: int = 1
    rollout_ep: int = 1                  # ranks of one engine that split the experts (attention replicated)
    rollout_batch_size: int = 8          # prompts per rollout step (global)
    prompt_len: int = 64
    max_response_len: int = 64
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    rm_type: str = "parity"
    eos_token_id: Optional[int] = None
    kv_blocks: int = 512
    kv_block_size: int = 16
    max_running: int = 256
    max_prefill_tokens: int = 16384
    use_cuda_graph: bool = True
    engine_memory_saver: Optional[bool] = None      # None: the engine's default (environment switch)
    seed: int = 0
    rollout_seed: int = 42
    offload_train: bool = False
    offload_rollout: bool = True
    # also free the rollout parameter buffer and the trainer's gradient buffer while the other
    # role runs (they are rewritten by the weight sync / zeroed before backward anyway)
    release_rollout_weights: bool = False
    pinned_prompts: bool = False
    # fuse tensor-parallel GEMMs with their collectives over NVLink peer memory (needs all ranks of a
    # TP group on one node); the symmetric workspace is allocated once per TP group
    fused_tp: bool = True
    fused_workspace_mb: int = 512
    num_prompts: int = 1 << 14
    # directory for per-step rollout dumps (rollout_<id>.jsonl, read by relax_b200.utils.visualize); engine-replica
    # rank 0 of data-parallel rank 0 writes its own samples
    save_debug_rollout_data: Optional[str] = None
    # held-out evaluation: rollout.evaluation.EvalDataset objects, run every `eval_interval` steps (and before the
    # first one unless `skip_eval_before_train`) with these sampling settings
    # user code by path ("pkg.mod:fn" or "/file.py:fn"): generate(engine, samples, sampling_params) -> samples fills
    # tokens / response_length / rollout_log_probs / status itself (multi-turn, tool use); reward(sample) -> float | dict
    custom_generate_function_path: Optional[str] = None
    speculative: bool = False            # the engine drafts with the model's MTP block (rollout/speculative.py)
    speculative_steps: int = 1           # proposals per verify pass
    rollout_global_dataset: bool = True             # False: no prompt dataset; the rollout function brings its own data
    rollout_function_path: Optional[str] = None     # user code that produces the whole rollout batch (see _run_rollout_function)
    # engines started by somebody else (``serve engine``): "host:port" each; engine replica r of this job uses its share
    # of the list (--rollout-external / --rollout-external-engine-addrs)
    rollout_external_addrs: Optional[Sequence[str]] = None
    # elastic pool over external engines: control endpoints on this port (+ engine replica index), autoscaling rules,
    # further servers that may be brought in, and the scale-out / scale-in knobs
    elastic_control_port: Optional[int] = None
    autoscaler_config: Optional[str] = None
    autoscaler_interval_s: float = 15.0
    rollout_standby_addrs: Optional[Sequence[str]] = None
    scale_out_timeout_s: float = 1800.0
    scale_in_drain_timeout_s: float = 300.0
    scale_weight_sync_precheck: bool = False
    scale_out_policy: str = "keep_partial"
    dynamic_sampling_filter_path: Optional[str] = None     # fn(group) -> bool | FilterOutput
    over_sampling_batch_size: Optional[int] = None         # groups generated per round while filtering (global)
    # partial rollout (relax/engine/rollout/sglang_rollout.py generate_rollout_async / abort): over-sampled groups
    # still running when the batch is full are aborted, kept with their partial responses in the rollout buffer and
    # continued by the next rollout step
    lora_adapter_mode: bool = False              # LoRA: sync the factors only, the engine applies them at run time
    opd_teacher_urls: Optional[list] = None      # remote teachers (POST <url>/score) scored before every training step
    partial_rollout: bool = False
    mask_offpolicy_in_partial_rollout: bool = False        # resumed samples: tokens of earlier policies leave the loss
    partial_rollout_max_aborted_count: Optional[int] = None  # a sample aborted more often is dropped with its group
    buffer_filter_path: Optional[str] = None               # fn(buffer, n) -> groups taken from the rollout buffer
    stop_token_ids: tuple = ()
    stop_strings: tuple = ()        # --rollout-stop: the response ends with the first of these strings (needs a codec)
    critic_lr: Optional[float] = None
    # rollout recovery (--use-health-check): a generate call that raises is retried after the engine's requests are
    # aborted, its cache flushed and the weights re-synchronised; after this many consecutive failures the error is raised
    use_health_check: bool = False
    max_consecutive_failures: int = 3
    num_critic_only_steps: int = 0      # PPO: the first rollouts train the critic alone
    critic_train_only: bool = False     # PPO: never update the policy (critic pre-training runs)
    # more user hooks by path: fn(samples) -> (raw_rewards, shaped_rewards) replaces reward normalisation;
    # fn(args_like, samples) marks samples with remove_sample = True (their loss mask is zeroed);
    # fn(args_like, samples) may rewrite the samples of a rollout before they are converted
    custom_reward_post_process_path: Optional[str] = None
    defer_reward_to_post_process: bool = False      # samples are not scored when they finish; the post-process scores the batch
    rollout_sample_filter_path: Optional[str] = None
    rollout_data_postprocess_path: Optional[str] = None
    log_passrate: bool = False                      # rollout/pass@k over the training groups (reward > 0.5 = correct)
    save_debug_train_data: Optional[str] = None     # directory: the training batch of every step as train_<id>.pt
    load_debug_rollout_data: Optional[str] = None   # directory of rollout_<id>.jsonl dumps replayed instead of generating
    # prompts from JSONL files instead of synthetic ids; `codec` (data.tokenizer) turns prompts into ids and responses
    # back into the text that rule rewards read
    prompt_data: Optional[str] = None
    input_key: str = "prompt"
    label_key: Optional[str] = "label"
    metadata_key: str = "metadata"
    tool_key: Optional[str] = None      # row field with tool definitions, rendered by the chat template
    multimodal_keys: Optional[dict] = None   # {"image": row field with the image path(s)}; needs a vision-language model
    rollout_shuffle: bool = False
    use_streaming_dataset: bool = False     # read the prompt files lazily through a shuffle buffer
    streaming_buffer_size: int = 1024
    codec: Optional[object] = None
    apply_chat_template: bool = False
    apply_chat_template_kwargs: dict = field(default_factory=dict)
    system_prompt: Optional[str] = None
    custom_rm_path: Optional[str] = None
    eval_datasets: list = field(default_factory=list)
    eval_interval: Optional[int] = None
    skip_eval_before_train: bool = False
    eval_temperature: float = 0.0
    eval_max_response_len: Optional[int] = None
    eval_reward_key: Optional[str] = None


class ColocatedGRPO:
    def __init__(self, cfg: ColocateConfig, device="cpu"):
        self.cfg = cfg
        self.device = torch.device(device)
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        ttp, tcp, tpp = cfg.trainer_tp, cfg.trainer_cp, cfg.trainer_pp
        dp = self.world // (ttp * tcp * tpp)
        if tpp > 1 and (tcp != 1 or cfg.rollout_tp != ttp):
            raise NotImplementedError("a pipeline-parallel trainer is colocated with engines of the same TP size, without CP")
        tep, rep_ = cfg.trainer_ep, cfg.rollout_ep
        if tep > 1 or rep_ > 1:
            if not (ttp == 1 and tcp == 1 and tpp == 1 and cfg.rollout_tp == 1 and tep == rep_):
                raise NotImplementedError("expert parallelism is colocated as trainer TP 1 x EP n with engines of EP n on the same ranks")
        if self.world > 1:
            self.ps = init_parallel_state(ParallelDims(tp=ttp, cp=tcp, dp=dp, pp=tpp, ep=tep))
        else:
            self.ps = single_process_state()
        # rollout engines: consecutive blocks of rollout_tp (or rollout_ep) ranks
        rtp = cfg.rollout_tp
        span = rtp * rep_
        self.num_engines = self.world // span
        self.engine_id = self.rank // span
        eng_group = None
        eng_ranks = tuple(range(self.engine_id * span, (self.engine_id + 1) * span))
        if span > 1:
            for e in range(self.num_engines):
                rr = list(range(e * span, (e + 1) * span))
                g = dist.new_group(rr)
                if e == self.engine_id:
                    eng_group = g
        eng_info = GroupInfo(eng_group, eng_ranks, self.rank % span)
        self.rollout_ep_group = eng_info if rep_ > 1 else None
        self.rollout_tp_group = eng_info if rep_ == 1 else GroupInfo(None, (self.rank,), 0)
        self.fused_comms = []
        if cfg.fused_tp and self.device.type == "cuda":
            from ..ops import fused_comm
            from ..parallel.symm_mem import attach_group

            for g in (self.rollout_tp_group, self.ps.tp):
                if fused_comm.comm_of(g) is None:
                    c = attach_group(g, self.device, cfg.fused_workspace_mb)
                    if c is not None:
                        self.fused_comms.append(c)

        self.teacher_pool = None
        if cfg.opd_teacher_urls:
            from ..algo.opd import HTTPTeacher, TeacherPool

            self.teacher_pool = TeacherPool([HTTPTeacher(u) for u in cfg.opd_teacher_urls])
        need_ref = cfg.train.loss.use_kl_loss or cfg.train.kl_coef != 0
        cfg.train.n_samples_per_prompt = cfg.train.n_samples_per_prompt
        self.actor = TrainActor(cfg.model, cfg.train, self.ps, device=device, seed=cfg.seed, with_reference=need_ref)
        # PPO: a value model of the same shape on the same ranks (relax/components/critic.py; separate optimizer and
        # learning rate), scored before and trained after every policy update
        self.critic = None
        if cfg.train.advantage_estimator in ("ppo", "gae"):
            from dataclasses import replace as _replace

            ccfg = _replace(cfg.train, optim=_replace(cfg.train.optim, lr=cfg.critic_lr or cfg.train.optim.lr), lora=None)
            self.critic = TrainActor(_replace(cfg.model, value_head=True, mtp_num_layers=0), ccfg, self.ps, device=device,
                                     seed=cfg.seed + 1, role="critic")
        if cfg.release_rollout_weights and self.actor.optimizer is not None:
            self.actor.optimizer.release_grads()   # before the engine allocates its weights and KV cache
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
        self.external = bool(cfg.rollout_external_addrs)
        if self.external:
            from ..rollout.external import ExternalEngine

            addrs = list(cfg.rollout_external_addrs)
            if cfg.rollout_tp != 1 or cfg.rollout_ep != 1:
                raise ValueError("external engines are addressed one per engine replica: --rollout-num-gpus-per-engine 1")
            if len(addrs) % self.num_engines:
                raise ValueError(f"{len(addrs)} external engine addresses do not divide over {self.num_engines} engine replicas")
            if cfg.partial_rollout or cfg.train.use_rollout_routing_replay or cfg.lora_adapter_mode:
                raise ValueError("partial rollout, rollout routing replay and adapter-mode LoRA sync need an in-process engine")
            k = len(addrs) // self.num_engines
            self.engine = ExternalEngine(cfg.model, addrs[self.engine_id * k:(self.engine_id + 1) * k], device, self.actor.model.dtype,
                                         max_model_len=cfg.prompt_len + cfg.max_response_len)
            self.elastic = None
            if cfg.elastic_control_port is not None or cfg.autoscaler_config:
                from ..rollout.elastic_service import ElasticControlServer
                from ..rollout.external import external_pool

                pool = external_pool(self.engine, cfg.rollout_standby_addrs or (), precheck=cfg.scale_weight_sync_precheck)
                self.elastic = ElasticControlServer(
                    pool, port=(cfg.elastic_control_port + self.engine_id) if cfg.elastic_control_port else 0,
                    autoscaler_config=cfg.autoscaler_config, metrics_fn=self.engine.server_metrics,
                    scale_out_timeout_s=cfg.scale_out_timeout_s, policy=cfg.scale_out_policy,
                    autoscale_interval_s=cfg.autoscaler_interval_s if cfg.autoscaler_config else 0.0)
                self.elastic.default_drain_s = cfg.scale_in_drain_timeout_s
        else:
            self.engine = RolloutEngine(cfg.model, self.rollout_tp_group, device=device, dtype=self.actor.model.dtype,
                                        num_kv_blocks=cfg.kv_blocks, block_size=cfg.kv_block_size,
                                        max_running=cfg.max_running, seed=cfg.rollout_seed + self.engine_id,
                                        max_prefill_tokens=cfg.max_prefill_tokens, use_cuda_graph=cfg.use_cuda_graph,
                                        memory_saver=cfg.engine_memory_saver,
                                        max_model_len=cfg.prompt_len + cfg.max_response_len,
                                        eos_token_id=cfg.eos_token_id, ep=self.rollout_ep_group,
                                        return_routed_experts=cfg.train.use_rollout_routing_replay, speculative=cfg.speculative,
                                        speculative_steps=cfg.speculative_steps)
        if cfg.model.vision is not None:
            # colocated: the engine embeds images with the trainer's tower itself (same parameters, nothing to sync)
            self.engine.attach_vision(self.actor.model.vision)
        if cfg.speculative and self.external:
            raise ValueError("speculative decoding runs in the in-process engine")

        def _plan(layout, r_tp, r_ep):
            """None (the default plan) unless the engine also needs the MTP block's weights."""
            if not cfg.speculative:
                return None
            from ..weight_sync.plan import build_plan

            return build_plan(cfg.model, layout, r_tp, r_ep, mtp=True)

        # the trainer replica that feeds my engine is the one I belong to (colocated)
        my_dp = self.ps.dp.rank
        tr_ranks = [r for r in self.ps.tp.ranks]
        if tpp > 1:
            # my replica spans tpp stages of ttp ranks; at every stage position sits one engine, and each engine needs
            # the layers of ALL stages: one sync object per engine of the replica, walked in the same order everywhere
            grid = {(st, j): j + ttp * (my_dp + dp * st) for st in range(tpp) for j in range(ttp)}
            self.syncs = []
            for st in range(tpp):
                er = [grid[(st, j)] for j in range(ttp)]
                self.syncs.append((WeightSync(cfg.model, TrainerLayout(tp=ttp, pp=tpp), rtp, grid, er,
                                              plan=_plan(TrainerLayout(tp=ttp, pp=tpp), rtp, 1)), tuple(er) == eng_ranks))
            self.sync = next(sy for sy, mine in self.syncs if mine)
            self._aligned = False
        elif tep > 1:
            self.sync = WeightSync(cfg.model, TrainerLayout(tp=1, ep=tep), 1, [self.rank], list(eng_ranks), rollout_ep=rep_,
                                   plan=_plan(TrainerLayout(tp=1, ep=tep), 1, rep_),
                                   aligned_ep_rank=self.ps.ep.rank)
            self.syncs = [(self.sync, True)]
            self._aligned = False        # the ranks of one engine generate the same samples: rows are re-split over DP
        else:
            self.sync = WeightSync(cfg.model, TrainerLayout(tp=ttp), rtp, tr_ranks, list(eng_ranks), plan=_plan(TrainerLayout(tp=ttp), rtp, 1))
            self.syncs = [(self.sync, True)]
            # with context parallelism a trainer replica spans tp x cp ranks that must all see the SAME rows (each holds
            # a slice of every sequence), while each of them feeds an engine of its own: rows always travel
            self._aligned = ttp == rtp and tuple(tr_ranks) == eng_ranks and tcp == 1
        self.adapter_syncs, self._base_synced = [], False
        if cfg.lora_adapter_mode and cfg.train.lora is not None:
            # adapter-mode LoRA sync (relax/backends/megatron/weight_update/lora_adapter_sync.py): the engine keeps the
            # base weights from the first sync and applies the factors at run time; later syncs move the factors only
            if tpp > 1 or tep > 1:
                raise NotImplementedError("LoRA adapter-mode sync covers tensor-parallel dense layouts (pp = ep = 1)")
            from ..weight_sync.plan import build_adapter_plan

            lo = cfg.train.lora
            plan = build_adapter_plan(cfg.model, TrainerLayout(tp=ttp), rtp, lo.rank, lo.target_modules)
            self.adapter_syncs = [(WeightSync(cfg.model, TrainerLayout(tp=ttp), rtp, tr_ranks, list(eng_ranks), plan=plan), True)]
            self.engine.weights.enable_lora(lo.rank, lo.scale, lo.target_modules)
        if not self._aligned and tpp == 1 and not (ttp == 1 or rtp == 1 or ttp == rtp):
            raise NotImplementedError("colocated sync needs trainer TP group == rollout engine ranks, or TP 1 on one side")
        self.queue = tq.init({"capacity_partitions": 2})
        ds = None
        if not cfg.rollout_global_dataset:
            from ..rollout.data_source import ShellDataSource

            if not cfg.rollout_function_path:
                raise ValueError("--disable-rollout-global-dataset leaves the prompts to user code: set --rollout-function-path")
            self.codec = cfg.codec
            self.data_source = ShellDataSource(cfg.train.n_samples_per_prompt)
        elif cfg.prompt_data:
            from ..data.tokenizer import ByteCodec, PromptEncoder
            from ..rollout.data_source import JsonlPromptDataset

            self.codec = cfg.codec or ByteCodec(cfg.model.vocab_size)
            enc = PromptEncoder(self.codec, cfg.apply_chat_template, cfg.apply_chat_template_kwargs, cfg.system_prompt, cfg.prompt_len)
            if cfg.use_streaming_dataset:
                from ..rollout.data_source import StreamingRolloutDataSource

                ds = None
                self.data_source = StreamingRolloutDataSource(cfg.prompt_data, enc, cfg.train.n_samples_per_prompt, cfg.streaming_buffer_size,
                                                              cfg.rollout_seed, cfg.input_key, cfg.label_key, cfg.metadata_key,
                                                              shuffle=cfg.rollout_shuffle)
            else:
                image_key = (cfg.multimodal_keys or {}).get("image")
                if image_key and cfg.model.vision is None:
                    raise ValueError(f"--multimodal-keys names images but model {cfg.model.name} has no vision tower")
                mmc = None
                if image_key:
                    from ..data.multimodal import MultimodalConfig

                    v = cfg.model.vision
                    mmc = MultimodalConfig(patch_size=v.patch_size, spatial_merge_size=v.spatial_merge_size,
                                           temporal_patch_size=v.temporal_patch_size)
                ds = JsonlPromptDataset(cfg.prompt_data, enc, cfg.input_key, cfg.label_key, cfg.metadata_key, cfg.tool_key,
                                        image_key=image_key, image_token_id=cfg.model.image_token_id if image_key else None,
                                        multimodal_config=mmc)
                if len(ds) == 0:
                    raise ValueError(f"no usable prompt in {cfg.prompt_data} (limit {cfg.prompt_len} tokens)")
        else:
            self.codec = cfg.codec
            if cfg.model.vision is not None:      # synthetic image prompts: text, one 8 x 8-patch image, text
                from ..rollout.data_source import SyntheticImagePromptDataset

                v = cfg.model.vision
                side = 4 * v.spatial_merge_size
                n_img = side * side // v.spatial_merge_size ** 2
                ds = SyntheticImagePromptDataset(cfg.num_prompts, max(1, (cfg.prompt_len - n_img) // 2), cfg.model.vocab_size,
                                                 cfg.model.image_token_id, (side, side),
                                                 v.in_channels * v.temporal_patch_size * v.patch_size ** 2,
                                                 v.spatial_merge_size, seed=cfg.seed)
            else:
                ds = SyntheticPromptDataset(cfg.num_prompts, cfg.prompt_len, cfg.model.vocab_size, seed=cfg.seed)
        if ds is not None:
            if cfg.partial_rollout or cfg.buffer_filter_path:
                from ..rollout.custom_generate import load_function as _lf
                from ..rollout.data_source import RolloutDataSourceWithBuffer

                bf = _lf(cfg.buffer_filter_path, 2, "rollout buffer filter") if cfg.buffer_filter_path else None
                self.data_source = RolloutDataSourceWithBuffer(ds, cfg.train.n_samples_per_prompt, shuffle=cfg.rollout_shuffle,
                                                               seed=cfg.rollout_seed, buffer_filter=bf)
            else:
                self.data_source = RolloutDataSource(ds, cfg.train.n_samples_per_prompt, shuffle=cfg.rollout_shuffle, seed=cfg.rollout_seed)
        from ..rollout.custom_generate import load_function, load_generate_function

        self.reward_fn = load_function(cfg.custom_rm_path, 1, "reward function") if cfg.custom_rm_path \
            else get_reward_spec(cfg.rm_type).fn
        if cfg.defer_reward_to_post_process:
            # relax/utils/arguments.py:2381-2390: with --rm-type dummy and a post-process function that owns the grader
            # (wakes it, scores the whole batch, puts it back to sleep) nothing is scored sample by sample
            if not cfg.custom_reward_post_process_path:
                raise ValueError("--defer-reward-to-post-process needs --custom-reward-post-process-path (the function that scores the batch)")
            self.reward_fn = lambda s: 0.0
        self.custom_generate = load_generate_function(cfg.custom_generate_function_path, None)
        self.rollout_function = load_function(cfg.rollout_function_path, 3, "rollout function") if cfg.rollout_function_path else None
        self.group_filter = load_function(cfg.dynamic_sampling_filter_path, 1, "group filter") \
            if cfg.dynamic_sampling_filter_path else None
        self.sampling_stats: dict = {}
        self.recoveries = 0
        self.reward_post_process = load_function(cfg.custom_reward_post_process_path, 1, "reward post-process") \
            if cfg.custom_reward_post_process_path else None
        self.sample_filter = load_function(cfg.rollout_sample_filter_path, 2, "sample filter") if cfg.rollout_sample_filter_path else None
        self.data_postprocess = load_function(cfg.rollout_data_postprocess_path, 2, "rollout post-process") \
            if cfg.rollout_data_postprocess_path else None
        self.timer = Timer()
        self.rollout_id = 0
        self.sync_weights()

    # user code by path: (attribute, configuration field, positional arguments it must take)
    RELOADABLE = (("custom_generate", "custom_generate_function_path", 3), ("rollout_function", "rollout_function_path", 3),
                  ("reward_fn", "custom_rm_path", 1), ("group_filter", "dynamic_sampling_filter_path", 1),
                  ("reward_post_process", "custom_reward_post_process_path", 1), ("sample_filter", "rollout_sample_filter_path", 2),
                  ("data_postprocess", "rollout_data_postprocess_path", 2))

    def reload_functions(self, names: Optional[Sequence[str]] = None) -> list:
        """Load the configured user functions again from their files, between two steps of a running job (an edited
        reward function or filter takes effect without a restart; relax/utils/reload_utils.py RELOADABLE_FUNCTIONS).
        Returns the attributes that were reloaded; a function that fails to load keeps its old version."""
        from ..rollout.custom_generate import reload_object

        done = []
        for attr, field_, npos in self.RELOADABLE:
            path = getattr(self.cfg, field_, None)
            if not path or (names is not None and attr not in names) or path.startswith("relax_b200."):
                continue
            if attr == "reward_fn" and self.cfg.defer_reward_to_post_process:
                continue
            try:
                fn = reload_object(path)
                if not callable(fn):
                    raise TypeError(f"{path} is not callable")
            except Exception as e:  # noqa: BLE001 - a broken edit must not take the run down
                import warnings

                warnings.warn(f"reload of {attr} from {path} failed, keeping the loaded version: {type(e).__name__}: {e}")
                continue
            setattr(self, attr, fn)
            done.append(attr)
        return done

    def close(self):
        """Collective over all ranks, before the process groups are destroyed: unmap the peers' symmetric buffers
        (tensor-parallel workspaces, the distributed optimizer's parameter / gradient buffers), meet, free this
        rank's, and destroy the engine sub-groups this object created."""
        from ..ops import fused_comm

        if self.device.type == "cuda":
            torch.cuda.synchronize()
        if getattr(self, "elastic", None) is not None:
            self.elastic.close()
        self.engine.close()        # graphs that captured NCCL operations must die before their communicator can
        for g in (self.rollout_tp_group, self.ps.tp):
            fused_comm.detach(g)
        for c in self.fused_comms:
            c.close()
        self.fused_comms = []
        for a in (self.actor, self.critic):
            for name in ("ep_comm", "cp_comm"):
                c = getattr(a, name, None) if a is not None else None
                if c is not None:
                    c.close()
                    setattr(a, name, None)
            opt = getattr(a, "optimizer", None) if a is not None else None
            if opt is not None and hasattr(opt, "close"):
                opt.close()
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    # ------------------------------------------------------------------ weight sync
    def sync_weights(self) -> float:
        adapter = self.cfg.lora_adapter_mode and self.cfg.train.lora is not None
        params = dict(self.actor.named_local_params(merged=not adapter))
        ms = 0.0
        if adapter and self._base_synced:
            # adapter mode after the first sync: the base weights on the engine are current, only the factors move
            for sync, mine in self.adapter_syncs:
                ms += sync.update_weights(params, self.engine.weights if mine else None, self.engine if mine else None,
                                          version=self.actor.weight_version)
            return ms
        for sync, mine in self.syncs:
            ms += sync.update_weights(params, self.engine.weights if mine else None, self.engine if mine else None,
                                      version=self.actor.weight_version)
        if adapter:
            for sync, mine in self.adapter_syncs:
                ms += sync.update_weights(params, self.engine.weights if mine else None, self.engine if mine else None,
                                          version=self.actor.weight_version)
            self._base_synced = True
        return ms

    # ------------------------------------------------------------------ rollout
    def _generate_with_recovery(self, prompts, sp, keys, images=None):
        if not self.cfg.use_health_check:
            return self.engine.generate(prompts, sp, group_keys=keys, images=images)
        failures = 0
        while True:
            try:
                return self.engine.generate(prompts, sp, group_keys=keys, images=images)
            except Exception as e:   # noqa: BLE001 - any engine failure takes the same recovery path
                failures += 1
                self.recoveries += 1
                if failures >= self.cfg.max_consecutive_failures:
                    raise RuntimeError(f"rollout engine failed {failures} times in a row") from e
                self.engine.abort_all()
                self.engine.flush_cache()
                self.sync_weights()

    def _generate_groups(self, n_groups: int, sp) -> list:
        """Draw ``n_groups`` prompt groups for this engine replica, generate and score them."""
        groups_all = self.data_source.get_samples(n_groups * self.num_engines)
        mine = groups_all[self.engine_id * n_groups:(self.engine_id + 1) * n_groups]
        flat = [s for g in mine for s in g]
        if self.custom_generate is not None:
            done = list(self.custom_generate(self.engine, flat, sp))
            for s in done:
                if s.reward is None:
                    s.reward = self.reward_fn(s)
            return mine
        images = [s.multimodal_train_inputs for s in flat] if any(s.multimodal_train_inputs for s in flat) else None
        res = self._generate_with_recovery([s.tokens for s in flat], sp, [s.group_index for s in flat], images)
        for s, r in zip(flat, res):
            self._fill_sample(s, r)
        return mine

    def _fill_sample(self, s, r, score: bool = True):
        """Copy a finished (or aborted) engine request into its sample and score it."""
        s.tokens = list(r.prompt) + list(r.output)
        s.response_length = len(r.output)
        s.rollout_log_probs = list(r.logprobs)
        s.weight_versions = sorted(set(list(s.weight_versions) + list(r.weight_versions)))
        if r.finish_reason == "abort":
            s.status = SampleStatus.ABORTED
        else:
            s.status = SampleStatus.TRUNCATED if r.finish_reason == "length" else SampleStatus.COMPLETED
        if r.routed_experts:
            s.rollout_routed_experts = r.routed_experts
        if self.codec is not None:
            if self.cfg.stop_strings and r.finish_reason != "abort":
                from ..data.tokenizer import cut_at_stop_strings

                n = cut_at_stop_strings(self.codec, list(r.output), self.cfg.stop_strings)
                if n is not None and n < len(r.output):      # generated past the stop string: drop the rest
                    s.tokens = list(r.prompt) + list(r.output[:n])
                    s.response_length, s.rollout_log_probs = n, list(r.logprobs[:n])
                    s.status = SampleStatus.COMPLETED
            s.response = self.codec.decode(s.tokens[len(s.tokens) - s.response_length:]) if s.response_length else ""
        if score and r.finish_reason != "abort":
            s.reward = self.reward_fn(s)

    def _generate_streaming(self, per: int, over: int, sp) -> list:
        """Over-sampled generation with early stop: ``over`` prompt groups are in flight, finished groups are scored
        and filtered as they complete, and once ``per`` groups are kept everything still running is aborted.  With
        ``partial_rollout`` the aborted groups go back to the rollout buffer with what they generated so far and the
        next rollout step continues them (their earlier tokens leave the loss with
        ``mask_offpolicy_in_partial_rollout``)."""
        from ..rollout.filters import FilterOutput

        cfg, eng = self.cfg, self.engine
        kept, inflight, by_rid = [], {}, {}
        stats = {"generated_groups": 0, "dropped_groups": 0, "rounds": 0, "aborted_samples": 0, "resumed_samples": 0}

        def close_group(g):
            out = self.group_filter(g) if self.group_filter is not None else FilterOutput(True)
            if out.keep if isinstance(out, FilterOutput) else bool(out):
                kept.append(g)
            else:
                stats["dropped_groups"] += 1
                why = getattr(out, "reason", None)
                if why:
                    stats[f"drop/{why}"] = stats.get(f"drop/{why}", 0) + 1

        def submit(n):
            stats["rounds"] += 1
            ds = self.data_source
            if hasattr(ds, "get_buffered"):      # my buffered (aborted) groups first, then my slice of fresh ones
                mine = ds.get_buffered(n)
                fresh = n - len(mine)
                if fresh:
                    mine += ds.get_fresh(fresh * self.num_engines)[self.engine_id * fresh:(self.engine_id + 1) * fresh]
            else:
                mine = ds.get_samples(n * self.num_engines)[self.engine_id * n:(self.engine_id + 1) * n]
            stats["generated_groups"] += len(mine)
            for g in mine:
                todo = 0
                for smp in g:
                    if smp.status in (SampleStatus.COMPLETED, SampleStatus.TRUNCATED) and smp.response_length:
                        continue          # finished before its group was aborted: keeps its response
                    n_prompt = len(smp.tokens) - smp.response_length
                    resumed = smp.response_length > 0
                    if resumed:
                        stats["resumed_samples"] += 1
                        smp.metadata["resumed_tokens"] = smp.response_length
                    im = smp.multimodal_train_inputs
                    rid = eng.add_request(smp.tokens[:n_prompt], sp, smp.group_index,
                                          resume_output=smp.tokens[n_prompt:] if resumed else None,
                                          resume_logprobs=smp.rollout_log_probs if resumed else None,
                                          **({k: im.get(k) for k in ("pixel_patches", "grid_thw", "image_embeds")} if im else {}))
                    by_rid[rid] = smp
                    todo += 1
                if todo:
                    inflight[g[0].group_index] = [g, todo]
                else:
                    close_group(g)

        submit(over)
        while len(kept) < per:
            if not eng.has_work:
                if stats["rounds"] >= 64:
                    raise RuntimeError(f"over-sampling: only {len(kept)}/{per} groups passed the filter after 64 rounds")
                submit(over)
                continue
            for r in eng.step():
                smp = by_rid.pop(r.rid)
                self._fill_sample(smp, r)
                n_old = smp.metadata.pop("resumed_tokens", 0)
                if n_old and cfg.mask_offpolicy_in_partial_rollout:
                    smp.loss_mask = [0] * n_old + [1] * (smp.response_length - n_old)
                ent = inflight[smp.group_index]
                ent[1] -= 1
                if ent[1] == 0:
                    del inflight[smp.group_index]
                    close_group(ent[0])
        surplus = kept[per:]
        # the batch is full: stop what is still running
        give_back = list(surplus)
        for r in eng.abort_all():
            smp = by_rid.pop(r.rid, None)
            if smp is None:
                continue
            self._fill_sample(smp, r, score=False)
            smp.metadata.pop("resumed_tokens", None)
            smp.abort_count += 1
            stats["aborted_samples"] += 1
        limit = cfg.partial_rollout_max_aborted_count
        for g, _ in inflight.values():
            if cfg.partial_rollout and (limit is None or all(x.abort_count <= limit for x in g)):
                give_back.append(g)
            else:
                stats["dropped_groups"] += 1
        if give_back:
            if hasattr(self.data_source, "buffer"):
                self.data_source.add_samples(give_back)
            else:
                stats["dropped_groups"] += len(give_back)
        self.sampling_stats = stats
        return kept[:per]

    def _run_rollout_function(self, rollout_id: int, per: int, sp) -> list[Sample]:
        """``--rollout-function-path``: user code produces the whole rollout batch of this engine replica
        (relax/utils/arguments.py:725-737: ``generate_rollout(args, rollout_id, data_source, evaluation=False)``).  The
        first argument here is a context object instead of the flag namespace, because the engine is a library object
        and not an HTTP address: ``ctx.engine``, ``ctx.sampling_params``, ``ctx.reward_fn``, ``ctx.codec``, ``ctx.cfg``,
        ``ctx.groups_wanted``, ``ctx.engine_id`` / ``ctx.num_engines``.  It returns prompt groups (lists of samples), a
        flat list of samples, or an object with a ``samples`` attribute holding either; every sample needs ``tokens``,
        ``response_length``, ``reward`` and ``status`` (a missing reward is filled by the reward function)."""
        from types import SimpleNamespace

        ctx = SimpleNamespace(engine=self.engine, sampling_params=sp, reward_fn=self.reward_fn, codec=self.codec, cfg=self.cfg,
                              groups_wanted=per, engine_id=self.engine_id, num_engines=self.num_engines)
        out = self.rollout_function(ctx, rollout_id, self.data_source, False)
        out = getattr(out, "samples", out)
        flat = [s for g in out for s in (g if isinstance(g, (list, tuple)) else [g])]
        n = self.cfg.train.n_samples_per_prompt
        if not flat or len(flat) % n:
            raise ValueError(f"the rollout function returned {len(flat)} samples; whole prompt groups of {n} are needed")
        for s in flat:
            if not s.tokens or not s.response_length:
                raise ValueError("the rollout function must set tokens and response_length on every sample")
            if s.reward is None:
                s.reward = self.reward_fn(s)
            if s.status == SampleStatus.PENDING:
                s.status = SampleStatus.COMPLETED
        self.sampling_stats = {}
        return flat

    def generate(self, rollout_id: int) -> list[Sample]:
        """One rollout batch.  With a group filter (``dynamic_sampling_filter_path``, e.g.
        ``relax_b200.rollout.filters:check_reward_nonzero_std``) the replica keeps generating
        ``over_sampling_batch_size`` groups at a time until its share of the batch passed the filter (DAPO dynamic
        sampling, relax/engine/rollout/sglang_rollout.py generate_rollout_async :763-1136)."""
        cfg = self.cfg
        per = cfg.rollout_batch_size // self.num_engines
        sp = SamplingParams(temperature=cfg.temperature, top_p=cfg.top_p, top_k=cfg.top_k,
                            max_new_tokens=cfg.max_response_len, stop_token_ids=tuple(cfg.stop_token_ids or ()))
        over_n = (cfg.over_sampling_batch_size or cfg.rollout_batch_size) // self.num_engines
        if self.rollout_function is not None:
            return self._run_rollout_function(rollout_id, per, sp)
        if self.custom_generate is None and not self.external and (cfg.partial_rollout or (self.group_filter is None and over_n > per)):
            groups = self._generate_streaming(per, max(per, over_n), sp)
        elif self.group_filter is None:
            groups = self._generate_groups(per, sp)
            self.sampling_stats = {}
        else:
            from ..rollout.filters import dynamic_sampling

            over = max(per, (cfg.over_sampling_batch_size or cfg.rollout_batch_size) // self.num_engines)
            groups, self.sampling_stats = dynamic_sampling(lambda n: self._generate_groups(n, sp), per, over, self.group_filter)
        return [s for g in groups for s in g]

    @property
    def _rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else 0

    def _load_dumped_rollout(self, rid: int) -> list[Sample]:
        """Replay a dumped rollout step (``--load-debug-rollout-data``): trainer-side debugging with the rollout
        engine out of the loop; tokens, rewards and rollout log-probs come from the file."""
        from ..utils.visualize import load_step

        _, rows = load_step(cfg_dir := self.cfg.load_debug_rollout_data, rid)
        out = []
        for r in rows:
            r = dict(r)
            st = r.pop("status", "completed")
            s = Sample(**{k: v for k, v in r.items() if k in Sample.__dataclass_fields__})
            s.status = SampleStatus(st)
            out.append(s)
        if not out:
            raise FileNotFoundError(f"no samples for rollout {rid} under {cfg_dir}")
        return out

    def _passrate(self, samples) -> dict:
        from ..rollout.evaluation import summarize

        groups: dict = {}
        for s in samples:
            groups.setdefault(s.group_index, []).append(s)
        m = summarize("train", list(groups.values()))
        return {k.replace("eval/train", "rollout/pass"): v for k, v in m.items() if "-pass@" in k}

    # ------------------------------------------------------------------ evaluation
    def evaluate(self) -> dict:
        """Evaluation rollout on every configured set with the current weights; engine replicas split nothing here
        (each runs the full sets: they are small) and report identical numbers."""
        from ..rollout.evaluation import evaluate as _eval

        cfg = self.cfg
        if cfg.offload_rollout:
            self.engine.resume_memory_occupation(("kv_cache",))
        sp = SamplingParams(temperature=cfg.eval_temperature, top_p=1.0, top_k=-1,
                            max_new_tokens=cfg.eval_max_response_len or cfg.max_response_len)
        with self.timer.span("eval"):
            m = _eval(self.engine, cfg.eval_datasets, self.reward_fn, sp, decode=self.codec.decode if self.codec is not None else None,
                      reward_key=cfg.eval_reward_key, generate_fn=self.custom_generate)
        if cfg.offload_rollout:
            self.engine.release_memory_occupation(("kv_cache", "cuda_graph"))
        return m

    def _eval_due(self, rid: int) -> bool:
        cfg = self.cfg
        if not cfg.eval_datasets or not cfg.eval_interval:
            return False
        if rid == 0:
            return not cfg.skip_eval_before_train
        return rid % cfg.eval_interval == 0

    # ------------------------------------------------------------------ one step
    def step(self) -> dict:
        cfg, rid = self.cfg, self.rollout_id
        t_all = time.perf_counter()
        eval_metrics = self.evaluate() if self._eval_due(rid) else {}
        with self.timer.span("rollout"):
            if cfg.offload_rollout:
                self.engine.resume_memory_occupation(("kv_cache",))
            samples = self._load_dumped_rollout(rid) if cfg.load_debug_rollout_data else self.generate(rid)
            if cfg.offload_rollout:
                self.engine.release_memory_occupation(("kv_cache", "cuda_graph"))
            if cfg.save_debug_rollout_data and self._rank == 0:
                from ..utils.visualize import dump_rollout

                dump_rollout(cfg.save_debug_rollout_data, rid, samples, extra={"weight_version": self.actor.weight_version})
        if self.sample_filter is not None:
            self.sample_filter(cfg, samples)
        if self.data_postprocess is not None:
            samples = self.data_postprocess(cfg, samples) or samples
        pass_metrics = self._passrate(samples) if cfg.log_passrate else {}
        with self.timer.span("data"):
            batch = convert_samples_to_train_data(
                samples, advantage_estimator=cfg.train.advantage_estimator,
                n_samples_per_prompt=cfg.train.n_samples_per_prompt,
                rewards_normalization=cfg.train.rewards_normalization,
                grpo_std_normalization=cfg.train.grpo_std_normalization,
                custom_reward_post_process=self.reward_post_process)
            # ranks of one engine hold identical rows; only the rows of replicas that
            # differ from mine have to travel
            batch = self._exchange(batch)
            part = tq.partition_name(rid)
            self.queue.put(batch, part, custom_meta=custom_meta_rows(batch), is_last=True)
            meta = self.queue.get_meta(list(batch.keys()), None, part, "actor")
            data = self.queue.get_data(meta)
        with self.timer.span("train"):
            if cfg.release_rollout_weights:
                self.engine.release_memory_occupation(("weights",))
                self.actor.optimizer.allocate_grads()
            if cfg.offload_train:
                self.actor.wake_up()
            if self.critic is not None:
                data["values"] = self.critic.compute_values(data)["values"]
            if cfg.save_debug_train_data:
                os.makedirs(cfg.save_debug_train_data, exist_ok=True)
                torch.save({k: v for k, v in data.items()}, os.path.join(cfg.save_debug_train_data, f"train_{rid}_rank{self._rank}.pt"))
            if self.teacher_pool is not None and data.get("teacher_log_probs") is None:
                with self.timer.span("teacher_log_probs"):
                    data["teacher_log_probs"] = self.teacher_pool.score(data)
            m = self.actor.train(rid, data, update_policy=not (self.critic is not None and (cfg.critic_train_only or rid < cfg.num_critic_only_steps)))
            self.actor.after_train()
            if self.critic is not None:       # `data` now carries the GAE returns computed with those values
                cm = self.critic.train_critic(rid, data)
                m.update({f"critic/{k}": v for k, v in cm.items()})
            if cfg.offload_train:
                self.actor.sleep()
            if cfg.release_rollout_weights:
                self.actor.optimizer.release_grads()
                self.engine.resume_memory_occupation(("weights",))
        self.queue.clear_partition(part)
        with self.timer.span("weight_sync"):
            sync_ms = self.sync_weights()
        n_resp = sum(batch["response_lengths"])
        n_tok = sum(batch["total_lengths"])
        st = self.engine.stats
        m.update(h2d_bytes=st.pop("h2d_bytes", 0), d2h_bytes=st.pop("d2h_bytes", 0) + 8 * len(m))
        m.update(weight_sync_ms=sync_ms, response_tokens_local=n_resp, total_tokens_local=n_tok,
                 raw_reward_mean=float(sum(batch["raw_reward"]) / max(1, len(batch["raw_reward"]))),
                 step_time=time.perf_counter() - t_all)
        m.update(self.timer.log_dict())
        m.update(eval_metrics)
        m.update(pass_metrics)
        if cfg.use_health_check:
            m["rollout/recoveries"] = float(self.recoveries)
        m.update({f"rollout/dynamic_sampling/{k}": float(v) for k, v in self.sampling_stats.items()})
        if getattr(self, "elastic", None) is not None:
            m["rollout/engines_active"] = float(len(self.elastic.pool.active()))
        if cfg.speculative:
            d, a_, v_ = (st.pop(k, 0) for k in ("spec_draft_tokens", "spec_accepted_tokens", "spec_verify_steps"))
            m.update({"rollout/spec_accept_rate": a_ / max(1, d), "rollout/spec_draft_tokens": float(d),
                      "rollout/spec_verify_steps": float(v_)})
        extra = getattr(self.custom_generate, "stats", None)        # a generate function may report its own gauges
        if callable(extra):
            m.update({k: float(v) for k, v in (extra() or {}).items()})
        self.rollout_id += 1
        return m

    def _exchange(self, batch: dict) -> dict:
        """Give every trainer replica the rows it trains on.  When engines and
        trainer replicas coincide nothing moves; otherwise rows are gathered
        and re-split evenly over data-parallel replicas."""
        if self.world == 1 or (self._aligned and not self.cfg.train.balance_data):
            return batch
        # one contributor per engine (its tp rank 0)
        leader = (self.rollout_ep_group.rank == 0) if self.rollout_ep_group is not None else (self.rollout_tp_group.rank == 0)
        contrib = batch if leader else None
        gathered = [None] * self.world
        dist.all_gather_object(gathered, contrib)
        merged: dict = {}
        for b in gathered:
            if b is None:
                continue
            for k, v in b.items():
                merged.setdefault(k, []).extend(v)
        return self.actor.split_for_dp(merged)
