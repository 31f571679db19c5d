"""relax_b200: asynchronous RL post-training for B200 (sm_100a) - trainer, rollout engine, weight sync, data plane and
orchestration in one package; the hot operators are hand-written CUDA in ``relax_b200/_C.so`` (built from ``csrc/``).

Entry points: ``python -m relax_b200.entrypoints.train`` (training), ``...entrypoints.serve`` (control-plane services),
``...entrypoints.visualize`` (rollout viewer); the Python API starts at :class:`relax_b200.orchestration.colocate.ColocatedGRPO`,
:class:`relax_b200.train.actor.TrainActor` and :class:`relax_b200.rollout.engine.RolloutEngine`.
"""
__version__ = "0.1.0"
