"""Controller: turns parsed flags into a running job.

It picks the execution mode (colocated synchronous RL, fully-async / hybrid role pipeline, SFT),
builds the model / trainer / rollout engine / data plane for it, resolves the start step from a
checkpoint, runs the training loop with periodic save / eval / metrics reporting, watches role
health, and shuts down gracefully on SIGTERM/SIGINT (finish the step in flight, save, exit).
The reference's controller does the same over Ray Serve deployments (relax/core/controller.py:
``__init__`` :147-212, ``training_loop`` :801-928, ``shutdown`` :930-959); here the roles are
objects of one process per GPU, wired by ``torch.distributed``.
"""
from __future__ import annotations

import os
import signal
import time
from typing import Optional

import torch
import torch.distributed as dist

from ..checkpoint import dist_ckpt
from ..config.arguments import model_config_from_args, train_config_from_args
from ..metrics.flops import B200_BF16_DENSE_TFLOPS, mfu, train_step_flops
from ..metrics.service import MetricsClient, MetricsService
from ..utils.profiler import TrainProfiler, memory_stats


def _get(a, name, default=None):
    v = getattr(a, name, None)
    return default if v is None else v


class Controller:
    def _codec(self, a):
        from ..data.tokenizer import build_codec

        if not (_get(a, "prompt_data", None) or _get(a, "eval_prompt_data", None) or _get(a, "rollout_stop", None)):
            return None
        return build_codec(_get(a, "hf_checkpoint", None), self.model_cfg.vocab_size)

    @staticmethod
    def _hf_post_hook(a):
        path = _get(a, "save_hf_post_hook_path", None)
        if not path:
            return None
        from ..rollout.custom_generate import load_function

        return load_function(path, 1, "HF export hook")

    def _eval_sets(self, a):
        return _eval_sets_from_args(a, self.model_cfg.vocab_size)

    def __init__(self, args, metrics: Optional[MetricsService] = None, device: Optional[str] = None):
        self.args = args
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        if device is None:
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}" if torch.cuda.is_available() else "cpu"
        self.device = device
        self.metrics = MetricsClient(service=metrics or MetricsService())
        self.model_cfg = model_config_from_args(args)
        self.train_cfg = train_config_from_args(args)
        if getattr(args, "lora_rank", 0):
            from ..train.lora import LoRAConfig

            kw = {}
            if _get(args, "lora_target_modules", None):
                tm = args.lora_target_modules
                kw["target_modules"] = tuple(tm.split(",")) if isinstance(tm, str) else tuple(tm)
            self.train_cfg.lora = LoRAConfig(rank=args.lora_rank, alpha=float(_get(args, "lora_alpha", None) or 2.0 * args.lora_rank),
                                             dropout=float(_get(args, "lora_dropout", None) or 0.0), **kw)
        self.mode = self._pick_mode()
        self._stop = False
        self.profiler = TrainProfiler(_get(args, "profile_dir", args.save and os.path.join(args.save, "profile")),
                                      _get(args, "profile_step_start", -1), _get(args, "profile_step_end", -1), self.rank,
                                      with_stack=bool(_get(args, "profile_with_stack", False)),
                                      record_memory=bool(_get(args, "profile_with_memory", False) or _get(args, "record_memory_history", False)))
        from ..utils.profiler import MemorySnapshotter

        self.memory_snapshot = MemorySnapshotter(_get(args, "memory_snapshot_dir", None), _get(args, "memory_snapshot_num_steps", None),
                                                 self.rank)
        self.start_rollout_id = dist_ckpt.resolve_start_rollout_id(args.load, args.start_rollout_id)
        if _get(args, "use_agentic_rollout", False):
            # the launcher daemon is forked here, while this process is still small
            from ..data.tokenizer import build_codec
            from ..rollout import agent_pipeline

            agent_pipeline.configure(args, build_codec(_get(args, "hf_checkpoint", None), self.model_cfg.vocab_size))
        self.runner = self._build_runner()
        self._maybe_resume()
        self._setup_health()

    # ------------------------------------------------------------------ health / two-tier recovery
    def _setup_health(self):
        """``--use-fault-tolerance``: a health registry for the roles of this process and the manager that maps a
        failure to a restart tier (relax/core/controller.py:977-1257): stateless roles restart in place (engine
        re-created from the trainer's weights), actor / rollout failures - or a role that keeps failing - restart
        globally (latest checkpoint reloaded, engine flushed and re-synchronised), at most ``--max-global-restart``
        times before the run stops with an error."""
        a = self.args
        self.health = self.health_mgr = None
        self.restarts = {"inplace": 0, "global": 0}
        self._fatal = None
        if not _get(a, "use_fault_tolerance", False):
            return
        from ..health.monitor import HealthManager, HealthRegistry

        self.health = HealthRegistry(heartbeat_timeout=float(_get(a, "rollout_health_check_timeout", 30.0)) * 4)
        for role in ("actor", "rollout"):
            self.health.register(role)
        self.health_mgr = HealthManager(self.health, self._restart_inplace, self._restart_global, self._on_fatal,
                                        max_global_restart=int(_get(a, "max_global_restart", 3)))

    def _recover_engine(self):
        eng = getattr(self.runner, "engine", None)
        if eng is not None:
            eng.abort_all()
            eng.flush_cache()
        q = getattr(self.runner, "queue", None)
        if q is not None:
            for part in list(q.get_partition_list()):
                q.clear_partition(part)
        if hasattr(self.runner, "sync_weights"):
            self.runner.sync_weights()

    def _restart_inplace(self, role: str):
        self.restarts["inplace"] += 1
        self._recover_engine()

    def _restart_global(self, role: str):
        """Back to the last durable state: the newest checkpoint under ``--save`` / ``--load`` when there is one (the
        step counter follows it), else the weights in memory; then the engine is rebuilt from them."""
        a, actor = self.args, self._actor()
        self.restarts["global"] += 1
        src = next((d for d in (_get(a, "save", None), _get(a, "load", None))
                    if d and os.path.isdir(d) and dist_ckpt.read_latest_iteration(d) is not None), None)
        if src is not None and actor is not None:
            it = dist_ckpt.read_latest_iteration(src)
            dist_ckpt.load_checkpoint(src, self.model_cfg, actor.ps, actor.model, actor.optimizer)
            if hasattr(self.runner, "rollout_id"):
                self.runner.rollout_id = it + 1
        self._recover_engine()

    def _on_fatal(self, msg: str):
        self._fatal = msg

    def _agree_failed(self, failed: bool) -> bool:
        """A failure on any rank restarts every rank (the roles are SPMD)."""
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return failed
        dev = self.device if str(self.device).startswith("cuda") and dist.get_backend() == "nccl" else "cpu"
        t = torch.tensor([1 if failed else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return bool(int(t[0]))

    def _guarded_step(self):
        """One runner step under the health manager.  Returns the step's metrics, or None after a recovery (the
        caller re-reads the step counter).  Only failures raised on the host between collectives can be recovered;
        a rank that dies inside a collective ends the job through the process-group timeout."""
        if self.health is None:
            return self.runner.step()
        multi = dist.is_initialized() and dist.get_world_size() > 1
        # between steps: a failure that any rank's monitors reported since the last step (an engine marked unhealthy, a
        # role that stopped beating) is agreed on by all ranks BEFORE anyone launches the next step, and all restart
        if self._agree_failed(bool(self.health.unhealthy())):
            if not self.health.unhealthy():
                self.health.report_error("rollout", "failure reported by another rank")
            return self._recover(None)
        err = None
        try:
            m = self.runner.step()
        except Exception as e:  # noqa: BLE001 - any role failure takes the recovery path
            import traceback

            where = "".join(traceback.format_tb(e.__traceback__))
            role = "rollout" if ("generate" in where or "rollout" in where and "train" not in where) else "actor"
            self.health.report_error(role, repr(e))
            if multi:
                # the other ranks are inside this step's collectives and cannot be called back from here: the job ends
                # (its launcher restarts it from the checkpoint); only a single-process job recovers in place
                raise
            err = e
        if err is None:
            step = getattr(self.runner, "rollout_id", 0)
            for role in ("actor", "rollout"):
                self.health.heartbeat(role, step)
            return m
        return self._recover(err)

    def _recover(self, err):
        self.health_mgr.check_once()
        if self._fatal is not None:
            raise RuntimeError(f"giving up after {self.health_mgr.global_restarts} global restarts: {self._fatal}") from err
        return None

    # ------------------------------------------------------------------ mode
    def _pick_mode(self) -> str:
        a = self.args
        if getattr(a, "loss_type", "policy_loss") in ("sft_loss", "seq_cls_loss"):
            return "sft"
        if getattr(a, "fully_async", False) or getattr(a, "hybrid", False):
            return "async"
        return "colocate"

    def _build_runner(self):
        a = self.args
        if self.mode == "colocate":
            from .colocate import ColocatedGRPO, ColocateConfig

            plen = _get(a, "rollout_max_prompt_len", 512)
            ctx = _get(a, "engine_context_length", None) or _get(a, "rollout_max_context_len", plen + a.rollout_max_response_len)
            page = _get(a, "engine_block_size", 16)
            cfg = ColocateConfig(
                model=self.model_cfg, train=self.train_cfg, trainer_tp=a.tensor_model_parallel_size,
                trainer_cp=a.context_parallel_size, trainer_pp=_get(a, "pipeline_model_parallel_size", 1),
                trainer_ep=_get(a, "expert_model_parallel_size", 1), rollout_ep=_get(a, "engine_ep", 1),
                rollout_tp=(_get(a, "rollout_num_gpus_per_engine", 1) if _get(a, "engine_ep", 1) == 1 else 1),
                rollout_batch_size=a.rollout_batch_size, prompt_len=plen,
                max_response_len=a.rollout_max_response_len, temperature=a.rollout_temperature,
                top_p=_get(a, "rollout_top_p", 1.0), top_k=_get(a, "rollout_top_k", -1), rm_type=a.rm_type or "parity",
                eos_token_id=getattr(self._codec(a), "eos_token_id", None),
                kv_blocks=_get(a, "kv_blocks", max(64, a.rollout_batch_size * a.n_samples_per_prompt * (ctx // 16 + 2))),
                kv_block_size=page if page > 1 else 16,
                max_running=_get(a, "engine_max_running", 256), max_prefill_tokens=_get(a, "engine_max_prefill_tokens", 16384),
                use_cuda_graph=not _get(a, "engine_disable_cuda_graph", False),
                engine_memory_saver=True if _get(a, "engine_memory_saver", False) else None, seed=a.seed, rollout_seed=a.rollout_seed,
                offload_rollout=a.offload_rollout, offload_train=a.offload_train,
                save_debug_rollout_data=_get(a, "save_debug_rollout_data", None),
                custom_generate_function_path=_get(a, "custom_generate_function_path", None),
                rollout_function_path=_get(a, "rollout_function_path", None),
                speculative=bool(_get(a, "engine_speculative_algorithm", None)),
                speculative_steps=int(_get(a, "engine_speculative_num_steps", 1) or 1),
                defer_reward_to_post_process=bool(_get(a, "defer_reward_to_post_process", False)),
                rollout_global_dataset=not bool(_get(a, "disable_rollout_global_dataset", False)),
                elastic_control_port=_get(a, "elastic_control_port", None), autoscaler_config=_get(a, "autoscaler_config", None),
                autoscaler_interval_s=float(_get(a, "autoscaler_interval", 15.0)),
                rollout_standby_addrs=_get(a, "rollout_standby_engine_addrs", None),
                scale_out_timeout_s=float(_get(a, "scale_out_timeout", 1800.0)),
                scale_in_drain_timeout_s=float(_get(a, "scale_in_drain_timeout", 300.0)),
                scale_weight_sync_precheck=bool(_get(a, "scale_weight_sync_precheck", False)),
                scale_out_policy={"keep": "keep_partial", "rollback": "rollback_all"}[_get(a, "scale_out_partial_success_policy", "keep")],
                rollout_external_addrs=(_get(a, "rollout_external_engine_addrs", None) if _get(a, "rollout_external", False) else None),
                custom_rm_path=_get(a, "custom_rm_path", None),
                prompt_data=_get(a, "prompt_data", None), input_key=_get(a, "input_key", None) or "prompt",
                label_key=_get(a, "label_key", None), metadata_key=_get(a, "metadata_key", None) or "metadata",
                tool_key=_get(a, "tool_key", None), multimodal_keys=_get(a, "multimodal_keys", None),
                rollout_shuffle=bool(_get(a, "rollout_shuffle", False)), codec=self._codec(a),
                use_streaming_dataset=bool(_get(a, "use_streaming_dataset", False)),
                streaming_buffer_size=_get(a, "streaming_buffer_size", None) or 1024,
                apply_chat_template=bool(_get(a, "apply_chat_template", False)),
                apply_chat_template_kwargs=_get(a, "apply_chat_template_kwargs", None) or {},
                system_prompt=_get(a, "system_prompt", None),
                dynamic_sampling_filter_path=_get(a, "dynamic_sampling_filter_path", None),
                over_sampling_batch_size=_get(a, "over_sampling_batch_size", None),
                opd_teacher_urls=_get(a, "opd_teacher_urls", None) if _get(a, "opd_type", None) else None,
                lora_adapter_mode=bool(_get(a, "lora_adapter_mode", False)),
                partial_rollout=bool(_get(a, "partial_rollout", False)),
                mask_offpolicy_in_partial_rollout=bool(_get(a, "mask_offpolicy_in_partial_rollout", False)),
                partial_rollout_max_aborted_count=_get(a, "partial_rollout_max_aborted_count", None),
                buffer_filter_path=_get(a, "buffer_filter_path", None),
                stop_token_ids=tuple(_get(a, "rollout_stop_token_ids", None) or ()),
                stop_strings=tuple(_get(a, "rollout_stop", None) or ()), critic_lr=_get(a, "critic_lr", None), use_health_check=bool(_get(a, "use_health_check", False)),
                max_consecutive_failures=_get(a, "rollout_health_check_max_consecutive_failures", None) or 3, num_critic_only_steps=_get(a, "num_critic_only_steps", 0) or 0, critic_train_only=bool(_get(a, "critic_train_only", False)),
                custom_reward_post_process_path=_get(a, "custom_reward_post_process_path", None),
                rollout_sample_filter_path=_get(a, "rollout_sample_filter_path", None),
                rollout_data_postprocess_path=_get(a, "rollout_data_postprocess_path", None),
                log_passrate=bool(_get(a, "log_passrate", False)), save_debug_train_data=_get(a, "save_debug_train_data", None),
                load_debug_rollout_data=_get(a, "load_debug_rollout_data", None),
                eval_datasets=self._eval_sets(a), eval_interval=_get(a, "eval_interval", None),
                skip_eval_before_train=bool(_get(a, "skip_eval_before_train", False)),
                eval_temperature=_get(a, "eval_temperature", None) or 0.0,
                eval_max_response_len=_get(a, "eval_max_response_len", None),
                eval_reward_key=_get(a, "eval_reward_key", None) or _get(a, "reward_key", None))
            run = ColocatedGRPO(cfg, device=self.device)
            if _get(a, "genrm_engine_addrs", None):
                # graders on their own engine servers (their own GPUs): nothing of theirs lives in this process
                from ..data.tokenizer import build_codec
                from ..rewards.genrm import build_remote_genrm

                gcodec = run.codec or build_codec(_get(a, "genrm_model_path", None) or _get(a, "hf_checkpoint", None), self.model_cfg.vocab_size)
                grm = build_remote_genrm(a.genrm_engine_addrs, gcodec)
                detok = run.codec.decode if run.codec is not None else (lambda ids: "")
                run.reward_fn, run.genrm = grm.reward_fn(detok), grm
            elif _get(a, "genrm_model_path", None):
                # generative reward model on in-house engines that share this rank's GPU (relax/components/genrm.py)
                from ..rewards.genrm import build_genrm

                grm = build_genrm(a.genrm_model_path, self.device, codec=run.codec, seed=a.seed)
                detok = run.codec.decode if run.codec is not None else (lambda ids: "")
                run.reward_fn, run.genrm = grm.reward_fn(detok), grm
            return run
        if self.mode == "sft":
            from ..train.actor import TrainActor
            from ..parallel.state import ParallelDims, init_parallel_state, single_process_state

            pp = _get(a, "pipeline_model_parallel_size", 1)
            ps = (init_parallel_state(ParallelDims(tp=a.tensor_model_parallel_size, cp=a.context_parallel_size, pp=pp,
                                                   dp=self.world // (a.tensor_model_parallel_size * a.context_parallel_size * pp)))
                  if self.world > 1 else single_process_state())
            role = "seq_cls" if getattr(a, "loss_type", None) == "seq_cls_loss" else "sft"
            if role == "seq_cls" and self.model_cfg.num_classes <= 0:
                raise ValueError("--loss-type seq_cls_loss needs --num-labels (the width of the classification head)")
            return _SFTRunner(TrainActor(self.model_cfg, self.train_cfg, ps, device=self.device, seed=a.seed, role=role), a)
        from .async_runner import build_async_runner

        return build_async_runner(self.args, self.model_cfg, self.train_cfg, self.device, self.start_rollout_id)

    # ------------------------------------------------------------------ checkpoints
    def _actor(self):
        return getattr(self.runner, "actor", None)

    def _load_hf_weights(self):
        """``--hf-checkpoint`` initialises the policy (unless a training checkpoint under ``--load`` takes over) and,
        with ``--ref-load`` pointing at a Hugging Face directory, the frozen reference snapshot."""
        from ..checkpoint import hf as H

        a, actor = self.args, self._actor()
        if actor is None:
            return
        src = _get(a, "hf_checkpoint", None)
        if src and "://" not in src and os.path.isdir(src) and not _get(a, "skip_hf_validate", False):
            H.validate_against_hf(self.model_cfg, src)
        if src and ("://" in src or H.is_hf_checkpoint(src)):
            H.load_hf_into_model(src, self.model_cfg, actor.ps, actor.model, strict=not _get(a, "only_load_weight", False))
            if actor.optimizer is not None:
                actor.optimizer.reload_master_from_params()
            if "ref" in actor.snapshots:
                actor.backup("ref")
            if hasattr(self.runner, "sync_weights"):
                self.runner.sync_weights()
        teacher = _get(a, "opd_teacher_load", None)
        if teacher and _get(a, "opd_type", None) and ("://" in teacher or H.is_hf_checkpoint(teacher)):
            # --opd-type megatron --opd-teacher-load <hf dir>: a teacher of the policy's shape kept as a weight snapshot
            keep = actor.param_buf.clone()
            H.load_hf_into_model(teacher, self.model_cfg, actor.ps, actor.model)
            actor.backup("teacher", to_host=actor.device.type == "cuda")
            actor.param_buf.copy_(keep)
        ref = _get(a, "ref_load", None)
        if ref and ref != src and ("://" in ref or H.is_hf_checkpoint(ref)) and "ref" in actor.snapshots:
            keep = actor.param_buf.clone()
            H.load_hf_into_model(ref, self.model_cfg, actor.ps, actor.model)
            actor.backup("ref", to_host=not actor.snapshots["ref"].is_cuda and actor.device.type == "cuda")
            actor.param_buf.copy_(keep)
        elif ref and ref != src and os.path.isdir(ref) and dist_ckpt.is_dist_checkpoint(ref) and "ref" in actor.snapshots:
            # --ref-load <training checkpoint dir> [--ref-ckpt-step N]: the reference is the policy of iteration N (default:
            # the latest) of another run (relax/backends/megatron/checkpoint.py loads the reference the same way)
            keep = actor.param_buf.clone()
            dist_ckpt.load_checkpoint(ref, self.model_cfg, actor.ps, actor.model, None, iteration=_get(a, "ref_ckpt_step", None))
            actor.backup("ref", to_host=not actor.snapshots["ref"].is_cuda and actor.device.type == "cuda")
            actor.param_buf.copy_(keep)

    def _maybe_resume(self):
        a, actor = self.args, self._actor()
        self._load_hf_weights()
        if not a.load or actor is None or not os.path.isdir(a.load):
            return
        if dist_ckpt.read_latest_iteration(a.load) is None:
            return
        skip_opt = _get(a, "no_load_optim", False) or _get(a, "reset_optimizer_states", False)
        dist_ckpt.load_checkpoint(a.load, self.model_cfg, actor.ps, actor.model, None if skip_opt else actor.optimizer)
        if hasattr(self.runner, "sync_weights"):
            self.runner.sync_weights()
        if hasattr(self.runner, "rollout_id"):
            self.runner.rollout_id = self.start_rollout_id
        critic = getattr(self.runner, "critic", None)
        cdir = _get(a, "critic_load", None) or a.load.rstrip("/") + "_critic"
        if critic is not None and os.path.isdir(cdir) and dist_ckpt.read_latest_iteration(cdir) is not None:
            dist_ckpt.load_checkpoint(cdir, critic.mcfg, critic.ps, critic.model,
                                      None if _get(a, "no_load_optim", False) else critic.optimizer)
        ds = getattr(self.runner, "data_source", None)
        it = dist_ckpt.read_latest_iteration(a.load)
        state_file = os.path.join(dist_ckpt.iter_dir(a.load, it), "rollout_data_source.json")
        if ds is not None and hasattr(ds, "load_state_dict") and os.path.exists(state_file):
            import json as _json

            with open(state_file) as f:
                ds.load_state_dict(_json.load(f))

    def save(self, rollout_id: int):
        a, actor = self.args, self._actor()
        if not a.save or actor is None:
            return
        dist_ckpt.save_checkpoint(a.save, rollout_id, self.model_cfg, actor.ps, actor.model,
                                  None if _get(a, "no_save_optim", False) else actor.optimizer)
        critic = getattr(self.runner, "critic", None)
        if critic is not None:      # PPO: the value model has its own checkpoint tree (--critic-save, default <save>_critic)
            cdir = _get(a, "critic_save", None) or a.save.rstrip("/") + "_critic"
            dist_ckpt.save_checkpoint(cdir, rollout_id, critic.mcfg, critic.ps, critic.model,
                                      None if _get(a, "no_save_optim", False) else critic.optimizer)
            if self.rank == 0:
                dist_ckpt.rotate_checkpoints(cdir, getattr(a, "max_checkpoints_to_keep", None))
        ds = getattr(self.runner, "data_source", None)
        if self.rank == 0 and ds is not None and hasattr(ds, "state_dict"):
            # where the prompt stream stands, so a resumed run goes on with the next unseen prompt
            import json as _json

            with open(os.path.join(dist_ckpt.iter_dir(a.save, rollout_id), "rollout_data_source.json"), "w") as f:
                _json.dump(ds.state_dict(), f)
        if self.rank == 0:
            dist_ckpt.rotate_checkpoints(a.save, getattr(a, "max_checkpoints_to_keep", None) or _get(a, "max_actor_ckpt_to_keep", None))
            if _get(a, "save_hf", None):       # also export Hugging Face files from the checkpoint just written
                from ..checkpoint import hf as H

                full = dist_ckpt.load_full_tensors(dist_ckpt.iter_dir(a.save, rollout_id))
                full = {k: v for k, v in full.items() if not k.startswith("optimizer.")}
                out = a.save_hf.format(rollout_id=rollout_id) if "{" in a.save_hf else os.path.join(a.save_hf, f"iter_{rollout_id:07d}")
                H.save_hf_checkpoint(out, self.model_cfg, H.convert_state_to_hf(self.model_cfg, full),
                                     quantize_fp8=_get(a, "save_hf_dtype", None) == "fp8",
                                     fp8_block=_get(a, "save_hf_fp8_block_size", None) or 128,
                                     post_hook=self._hf_post_hook(a))

    # ------------------------------------------------------------------ loop
    def _install_signal_handlers(self):
        def handler(signum, frame):
            self._stop = True

        for s in (signal.SIGTERM, signal.SIGINT):
            try:
                signal.signal(s, handler)
            except ValueError:   # not the main thread (tests)
                pass

        def reload_handler(signum, frame):       # kill -HUP <pid>: user functions are loaded again before the next step
            self._reload_requested = True

        try:
            signal.signal(signal.SIGHUP, reload_handler)
        except (ValueError, AttributeError):
            pass

    def training_loop(self) -> list:
        a = self.args
        self._install_signal_handlers()
        history = []
        if self.mode == "async":
            out = self.runner.run()
            for rid, m in out:
                self.metrics.log_metrics_batch(rid, {k: float(v) for k, v in m.items() if isinstance(v, (int, float))})
                self.metrics.report_step(rid)
            if out:
                self.save(max(r for r, _ in out))
            return out
        rid = self.start_rollout_id
        if _get(a, "timeline_dump_dir", None) and getattr(self.runner, "timer", None) is not None:
            self.runner.timer.record_timeline = True
            self.runner.timer.pid = self.rank
        if a.num_rollout is None and _get(a, "num_epoch", None) and hasattr(self.runner, "data_source"):
            # --num-epoch: as many rollouts as it takes to see every prompt that many times
            a.num_rollout = max(1, a.num_epoch * len(self.runner.data_source.dataset) // max(1, a.rollout_batch_size))
        ref_every = _get(a, "ref_update_interval", None)
        while rid < a.num_rollout and not self._stop:
            t0 = time.perf_counter()
            if getattr(self, "_reload_requested", False) and hasattr(self.runner, "reload_functions"):
                self._reload_requested = False
                print(f"[reload] user functions reloaded: {self.runner.reload_functions()}", flush=True)
            m = self._guarded_step()
            if m is None:                     # recovered from a failure: go on from where the restart left the job
                rid = getattr(self.runner, "rollout_id", rid)
                continue
            actor = self._actor()
            if ref_every and actor is not None and "ref" in actor.snapshots and (rid + 1) % ref_every == 0:
                # --ref-update-interval: the reference follows the policy every N rollouts
                actor.backup("ref", to_host=not actor.snapshots["ref"].is_cuda and actor.device.type == "cuda")
                m["ref_updated"] = 1.0
            dt = time.perf_counter() - t0
            rec = {k: float(v) for k, v in m.items() if isinstance(v, (int, float))}
            rec["perf/step_time"] = dt
            if "total_tokens_local" in m and getattr(a, "profile_with_flops", True):
                n = max(1, int(m["total_tokens_local"]))
                seq = _get(a, "rollout_max_prompt_len", 512) + a.rollout_max_response_len if self.mode == "colocate" else n
                lens = [seq] * max(1, n // max(1, seq))
                fl = train_step_flops(self.model_cfg, lens, forward_only_passes=2)
                rec["perf/train_mfu"] = mfu(fl, max(m.get("perf/train_time", dt), 1e-9), 1, B200_BF16_DENSE_TFLOPS)
            rec.update(memory_stats(self.device) if str(self.device).startswith("cuda") else {})
            self.metrics.log_metrics_batch(rid, rec)
            self.metrics.report_step(rid)
            self.profiler.step()
            self.memory_snapshot.step()
            history.append(rec)
            rid += 1
            if a.save and a.save_interval and rid % a.save_interval == 0:
                self.save(rid - 1)   # a checkpoint is named after the last rollout it contains
        if self._stop and a.save and rid > self.start_rollout_id:
            self.save(rid - 1)   # interrupted: keep what was learned
        self.profiler.close()
        self.memory_snapshot.close()
        tdir = _get(a, "timeline_dump_dir", None)
        timer = getattr(self.runner, "timer", None)
        if tdir and timer is not None and hasattr(timer, "dump_chrome_trace"):     # one Chrome trace of the phase spans per rank
            os.makedirs(tdir, exist_ok=True)
            timer.dump_chrome_trace(os.path.join(tdir, f"timeline_rank{self.rank}.json"))
        return history

    def shutdown(self):
        svc = self.metrics.service
        if svc is not None:
            svc.close()
        if hasattr(self.runner, "close"):
            self.runner.close()


class _SFTRunner:
    """One ``step()`` = one global batch of the streaming SFT dataset."""

    def __init__(self, actor, args):
        from ..data.sft import Prefetcher, StreamingSFTDataset, batches_with_cursor

        self.actor = actor
        files = [p for p in str(args.prompt_data).split(",") if p]
        from ..data.tokenizer import build_codec, has_tokenizer_files

        hf = _get(args, "hf_checkpoint", None)      # the model's own tokenizer when its files are there, bytes otherwise
        tok = build_codec(hf, actor.mcfg.vocab_size).encode if has_tokenizer_files(hf) else _byte_tokenizer(actor.mcfg.vocab_size)
        ds = StreamingSFTDataset(files, tok, actor.ps.dp.rank, actor.ps.dp.size,
                                 max_len=_get(args, "rollout_max_context_len", 4096), epochs=None)
        per_rank = max(1, actor.cfg.global_batch_size // actor.ps.dp.size)
        if actor.role == "seq_cls":
            self.batches = self._classification_batches(files, tok, per_rank, args)
        else:
            # batches are tokenised ahead of the step by a background thread (--sft-prefetch-buffer-size, counted in samples)
            depth = max(1, int(_get(args, "sft_prefetch_buffer_size", 64)) // per_rank)
            self._pairs = Prefetcher(batches_with_cursor(ds, per_rank), depth)
            self.batches = self._consume(self._pairs)
        self.dataset = ds
        self._cursor = ds.state_dict()
        self.data_source = self            # what the controller saves / restores next to a checkpoint
        self._init_eval(args, files, tok)
        self._init_predict(args, files, tok)

    def _consume(self, pairs):
        for batch, state in pairs:
            self._cursor = state
            yield batch

    def state_dict(self) -> dict:
        """Where the data stream stands after the last batch that was trained on."""
        return dict(self._cursor, steps=getattr(self, "steps", 0))

    def load_state_dict(self, st: dict):
        from ..data.sft import Prefetcher, batches_with_cursor

        if getattr(self, "_pairs", None) is None:
            return                       # classification batches restart from the top of their files
        self._pairs.close()
        self.dataset.load_state_dict(st)
        self._cursor = self.dataset.state_dict()
        self.steps = int(st.get("steps", 0))
        per_rank = max(1, self.actor.cfg.global_batch_size // self.actor.ps.dp.size)
        self._pairs = Prefetcher(batches_with_cursor(self.dataset, per_rank), self._pairs._q.maxsize)
        self.batches = self._consume(self._pairs)

    def _classification_batches(self, files, tok, per_rank, args):
        """``{"text" | "prompt": ..., "label": id | [ids] | multi-hot}`` rows -> batches with ``labels``
        (relax/engine/sft/ classification datasets): the whole text is context, the class head reads its last token."""
        import json

        actor = self.actor
        C = actor.mcfg.num_classes
        multi = (actor.cfg.problem_type == "multi_label_classification")
        key_in, key_lab = _get(args, "input_key", None) or "prompt", _get(args, "label_key", None) or "label"
        max_len = _get(args, "rollout_max_context_len", 4096)
        rows, n = [], 0
        while True:
            for path in files:
                with open(path, encoding="utf-8") as f:
                    for line in f:
                        if not line.strip():
                            continue
                        mine = n % actor.ps.dp.size == actor.ps.dp.rank
                        n += 1
                        if not mine:
                            continue
                        r = json.loads(line)
                        text = r.get(key_in) or r.get("prompt") or r.get("text") or ""
                        toks = tok(text)[:max_len] or [0]
                        lab = r[key_lab]
                        if multi:
                            ids = lab if isinstance(lab, (list, tuple)) else [lab]
                            lab = [float(x) for x in ids] if len(ids) == C and set(ids) <= {0, 1} else \
                                [1.0 if c in set(int(i) for i in ids) else 0.0 for c in range(C)]
                        else:
                            lab = int(lab)
                        rows.append((toks, lab))
                        if len(rows) == per_rank:
                            yield {"tokens": [t for t, _ in rows], "response_lengths": [1] * len(rows),
                                   "loss_masks": [[1]] * len(rows), "labels": [l for _, l in rows]}
                            rows = []

    def step(self) -> dict:
        b = next(self.batches)
        m = self.actor.train_seq_cls(b) if self.actor.role == "seq_cls" else self.actor.train_sft(b)
        m["total_tokens_local"] = sum(len(t) for t in b["tokens"])
        self.steps = getattr(self, "steps", 0) + 1
        if self.eval is not None and self.steps % self.eval["interval"] == 0:
            m.update(self.run_eval())
        if self.predict is not None and self.steps % self.predict["interval"] == 0:
            m.update(self.run_predict(self.steps))
        return m

    # ------------------------------------------------------------------ periodic evaluation
    def _eval_rows(self, args, files):
        """The evaluation rows: ``--eval-prompt-data`` (name path pairs) or a fixed-seed ``--eval-size`` subset of the
        training files (relax/engine/sft/runtime.py resolve_sft_eval_split / resolve_sft_split_indices)."""
        import json
        import random

        rows = []
        pairs = _get(args, "eval_prompt_data", None) or []
        paths = [pairs[i + 1] for i in range(0, len(pairs) - 1, 2)]
        for path in (paths or files):
            with open(path, encoding="utf-8") as f:
                rows += [json.loads(line) for line in f if line.strip()]
        if not paths:
            k = _get(args, "eval_size", None)
            if not k:
                return None
            rows = random.Random(int(_get(args, "seed", 0)) + 1234).sample(rows, min(int(k), len(rows)))
        return rows

    def _init_eval(self, args, files, tok):
        """``--eval-interval N`` under SFT: every N steps the held-out rows are scored without training on them -
        token-level NLL / perplexity over the assistant turns (relax/engine/sft/eval/ppl.py), or accuracy and macro-F1
        of the class head (relax/engine/sft/eval/classification.py)."""
        from ..data.sft import render_chat, to_train_sample

        self.eval = None
        n = _get(args, "eval_interval", None)
        rows = self._eval_rows(args, files) if n else None
        if not n or not rows:
            return
        actor = self.actor
        rows = rows[actor.ps.dp.rank::actor.ps.dp.size]
        max_len = _get(args, "rollout_max_context_len", 4096)
        if actor.role == "seq_cls":
            key_in, key_lab = _get(args, "input_key", None) or "prompt", _get(args, "label_key", None) or "label"
            toks = [(tok(r.get(key_in) or r.get("prompt") or r.get("text") or "")[:max_len] or [0]) for r in rows]
            batch = {"tokens": toks, "response_lengths": [1] * len(rows), "loss_masks": [[1]] * len(rows), "labels": [r[key_lab] for r in rows]}
        else:
            samples = []
            for r in rows:
                msgs = r.get("messages") or [{"role": "user", "content": r.get("prompt", "")}, {"role": "assistant", "content": r.get("response", "")}]
                smp = to_train_sample(*render_chat(msgs, tok), max_len=max_len)
                if smp is not None:
                    samples.append(smp)
            batch = {"tokens": [s_["tokens"] for s_ in samples], "response_lengths": [s_["response_length"] for s_ in samples],
                     "loss_masks": [s_["loss_mask"] for s_ in samples]}
        self.eval = {"interval": int(n), "batch": batch}

    def run_eval(self) -> dict:
        actor, batch = self.actor, self.eval["batch"]
        if actor.role != "seq_cls":
            return actor.evaluate_ppl(batch)
        C = actor.mcfg.num_classes
        logits = torch.stack([x.float() for x in actor.predict_classes(batch)]) if batch["tokens"] else torch.zeros(0, C)
        stats = torch.zeros(3, C, dtype=torch.float64, device=actor.device)           # tp, predicted, actual per class
        if actor.cfg.problem_type == "multi_label_classification":
            pred = torch.sigmoid(logits) > (actor.cfg.classification_threshold or 0.5)
            lab = torch.zeros_like(pred)
            for i, l_ in enumerate(batch["labels"]):
                ids = l_ if isinstance(l_, (list, tuple)) else [l_]
                hot = [bool(x) for x in ids] if len(ids) == C and set(ids) <= {0, 1} else [c in set(int(x) for x in ids) for c in range(C)]
                lab[i] = torch.tensor(hot, device=lab.device)
            correct = (pred == lab).all(-1).double().sum()
        else:
            cls = logits.argmax(-1)
            want = torch.tensor([int(l_) for l_ in batch["labels"]], device=cls.device)
            pred = torch.nn.functional.one_hot(cls, C).bool()
            lab = torch.nn.functional.one_hot(want, C).bool()
            correct = (cls == want).double().sum()
        stats[0], stats[1], stats[2] = (pred & lab).sum(0), pred.sum(0), lab.sum(0)
        tot = torch.stack([correct, torch.tensor(float(len(batch["tokens"])), dtype=torch.float64, device=actor.device)])
        if actor.ps.dp.size > 1:
            dist.all_reduce(stats, group=actor.ps.dp.group)
            dist.all_reduce(tot, group=actor.ps.dp.group)
        prec, rec = stats[0] / stats[1].clamp_min(1), stats[0] / stats[2].clamp_min(1)
        f1 = torch.where(prec + rec > 0, 2 * prec * rec / (prec + rec).clamp_min(1e-12), torch.zeros_like(prec))
        seen = stats[2] > 0
        return {"eval/accuracy": float(tot[0] / tot[1].clamp_min(1)), "eval/macro_f1": float(f1[seen].mean()) if bool(seen.any()) else 0.0,
                "eval/samples": float(tot[1])}

    # ------------------------------------------------------------------ periodic predict pass
    def _init_predict(self, args, files, tok):
        """``--sft-predict-interval N`` (relax/engine/sft/predict/loop.py, predict/runner.py): every N steps the current
        weights generate completions for the evaluation conversations - each cut before its last assistant turn,
        which becomes the reference - and the results go to ``<save>/predict/predictions_step_<step>.jsonl``.  The
        evaluation set is ``--eval-prompt-data`` (name path pairs) or a fixed-seed ``--eval-size`` subset of the
        training files.  The engine is built on first use and gives its KV cache back after every pass."""
        import json
        import random

        self.predict = None
        n = _get(args, "sft_predict_interval", None)
        if not n:
            return
        if not _get(args, "save", None):
            raise ValueError("--sft-predict-interval writes to <save>/predict/: set --save")
        if self.actor.ps.tp.size > 1 or self.actor.ps.pp.size > 1:
            raise NotImplementedError("the predict pass runs an engine next to a tp = pp = 1 trainer")
        rows = self._eval_rows(args, files)
        if not rows:
            raise ValueError("--sft-predict-interval needs --eval-prompt-data or --eval-size")
        conv = []
        for r in rows:
            msgs = r.get("messages") or [{"role": "user", "content": r.get("prompt", "")}, {"role": "assistant", "content": r.get("response", "")}]
            last = max((i for i, m_ in enumerate(msgs) if m_["role"] == "assistant"), default=-1)
            ref = msgs[last]["content"] if last >= 0 else ""
            conv.append((msgs[:last] if last >= 0 else msgs, ref if isinstance(ref, str) else json.dumps(ref, ensure_ascii=False)))
        self.predict = {"interval": int(n), "conv": conv, "tok": tok, "dir": os.path.join(args.save, "predict"),
                        "max_new": int(_get(args, "eval_max_response_len", None) or _get(args, "rollout_max_response_len", 64)),
                        "max_ctx": int(_get(args, "rollout_max_context_len", 4096)), "engine": None, "sync": None,
                        "hf": _get(args, "hf_checkpoint", None)}

    def run_predict(self, step: int) -> dict:
        import json
        import time as _time

        from ..data.sft import render_chat
        from ..data.tokenizer import build_codec
        from ..rollout.engine import RolloutEngine, SamplingParams
        from ..weight_sync.plan import TrainerLayout
        from ..weight_sync.sync import WeightSync

        P, actor = self.predict, self.actor
        t0 = _time.perf_counter()
        mine = P["conv"][actor.ps.dp.rank::actor.ps.dp.size]
        prompts = []
        for msgs, _ in mine:
            toks, _m = render_chat(msgs, P["tok"])
            prompts.append((toks + P["tok"]("<|assistant|>\n"))[-(P["max_ctx"] - P["max_new"]):])
        if P["engine"] is None:
            need = sum((len(p) + P["max_new"]) // 16 + 2 for p in prompts) + 8
            P["engine"] = RolloutEngine(actor.mcfg, device=actor.device, dtype=actor.model.dtype, num_kv_blocks=max(64, need), block_size=16,
                                        max_model_len=P["max_ctx"], use_cuda_graph=False, memory_saver=False)
            me = dist.get_rank() if dist.is_initialized() else 0
            P["sync"] = WeightSync(actor.mcfg, TrainerLayout(tp=1), 1, [me], [me])
            P["decode"] = build_codec(P["hf"], actor.mcfg.vocab_size).decode
        eng = P["engine"]
        eng.resume_memory_occupation(("kv_cache",))
        P["sync"].update_weights(dict(actor.named_local_params()), eng.weights, eng, version=step)
        out = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=P["max_new"]))
        eng.release_memory_occupation(("kv_cache", "cuda_graph"))
        os.makedirs(P["dir"], exist_ok=True)
        suffix = f"_rank{actor.ps.dp.rank}" if actor.ps.dp.size > 1 else ""
        path = os.path.join(P["dir"], f"predictions_step_{step}{suffix}.jsonl")
        with open(path, "w", encoding="utf-8") as f:
            for (msgs, ref), r in zip(mine, out):
                f.write(json.dumps({"step": step, "prompt": msgs, "reference": ref, "prediction": P["decode"](r.output),
                                    "finish_reason": r.finish_reason}, ensure_ascii=False) + "\n")
        return {"predict/samples": float(len(out)), "predict/time": _time.perf_counter() - t0,
                "predict/response_len": sum(len(r.output) for r in out) / max(1, len(out))}


def _eval_sets_from_args(a, vocab: int):
    pairs = getattr(a, "eval_prompt_data", None)
    if not pairs:
        return []
    import json as _json

    from ..rollout.evaluation import load_eval_datasets

    overrides = None
    if getattr(a, "eval_config", None):
        with open(a.eval_config) as f:
            overrides = _json.load(f)
    from ..data.tokenizer import PromptEncoder, build_codec

    enc = PromptEncoder(build_codec(getattr(a, "hf_checkpoint", None), vocab), bool(getattr(a, "apply_chat_template", False)),
                        getattr(a, "apply_chat_template_kwargs", None) or {}, getattr(a, "system_prompt", None))
    sets = load_eval_datasets(pairs, enc, getattr(a, "eval_input_key", None) or "prompt", getattr(a, "eval_label_key", None) or "label",
                              getattr(a, "n_samples_per_eval_prompt", 1), getattr(a, "eval_size", None),
                              getattr(a, "eval_max_prompt_len", None), overrides)
    for ds in sets:
        ds.top_p = ds.top_p if ds.top_p is not None else getattr(a, "eval_top_p", None)
        ds.top_k = ds.top_k if ds.top_k is not None else getattr(a, "eval_top_k", None)
    return sets


def _byte_tokenizer(vocab: int):
    """Fallback tokenizer when no HF tokenizer directory is given: UTF-8 bytes offset past the special ids."""
    return lambda s: [3 + (b % max(1, vocab - 3)) for b in s.encode("utf-8")]
