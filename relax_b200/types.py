"""Sample / batch schema shared by rollout, data plane and trainer.

Field set follows relax/utils/types.py:26-217 (``Sample``) and the train-batch
keys of relax/utils/utils.py:96-168.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field, asdict
from typing import Any, Optional


class SampleStatus(str, enum.Enum):
    PENDING = "pending"
    COMPLETED = "completed"
    TRUNCATED = "truncated"
    ABORTED = "aborted"
    FAILED = "failed"


@dataclass
class SpecInfo:
    spec_accept_token_num: int = 0
    spec_draft_token_num: int = 0
    spec_verify_ct: int = 0
    completion_token_num: int = 0

    @property
    def accept_rate(self) -> float:
        return self.spec_accept_token_num / max(1, self.spec_draft_token_num)


@dataclass
class PrefixCacheInfo:
    cached_tokens: int = 0
    total_prompt_tokens: int = 0

    @property
    def hit_rate(self) -> float:
        return self.cached_tokens / max(1, self.total_prompt_tokens)


@dataclass
class Sample:
    group_index: Optional[int] = None
    index: Optional[int] = None
    prompt: Any = ""
    tokens: list = field(default_factory=list)          # prompt + response token ids
    rollout_tokens: Optional[list] = None
    multimodal_inputs: Optional[dict] = None
    multimodal_train_inputs: Optional[dict] = None
    response: str = ""
    response_length: int = 0
    label: Any = None
    reward: Any = None
    custom_advantage: Optional[float] = None
    loss_mask: Optional[list] = None
    weight_versions: list = field(default_factory=list)
    rollout_log_probs: Optional[list] = None
    rollout_routed_experts: Any = None
    remove_sample: bool = False
    abort_count: int = 0
    teacher_log_probs: Optional[list] = None
    teacher_topk_ids: Any = None
    teacher_topk_log_probs: Any = None
    status: SampleStatus = SampleStatus.PENDING
    metadata: dict = field(default_factory=dict)
    generate_function_path: Optional[str] = None
    train_metadata: Optional[dict] = None
    session_id: Optional[str] = None
    non_generation_time: float = 0.0
    spec_info: SpecInfo = field(default_factory=SpecInfo)
    prefix_cache_info: PrefixCacheInfo = field(default_factory=PrefixCacheInfo)

    def to_dict(self) -> dict:
        d = asdict(self)
        d["status"] = self.status.value
        return d

    @staticmethod
    def from_dict(d: dict) -> "Sample":
        d = dict(d)
        d["status"] = SampleStatus(d.get("status", "pending"))
        d["spec_info"] = SpecInfo(**d.get("spec_info", {}))
        d["prefix_cache_info"] = PrefixCacheInfo(**d.get("prefix_cache_info", {}))
        return Sample(**d)

    def get_reward_value(self, key: Optional[str] = None) -> float:
        if isinstance(self.reward, dict):
            return float(self.reward[key or "score"])
        return float(self.reward)

    @property
    def prompt_length(self) -> int:
        return len(self.tokens) - self.response_length

    @property
    def effective_response_length(self) -> int:
        return sum(self.loss_mask) if self.loss_mask is not None else self.response_length


@dataclass
class ParamInfo:
    name: str
    dtype: Any
    shape: tuple
    attrs: dict
    size: int
    src_rank: int


# keys of a train batch (lists with one entry per sample row)
TRAIN_BATCH_KEYS = (
    "tokens", "response_lengths", "rewards", "raw_reward", "group_index", "truncated", "sample_indices",
    "loss_masks", "sample_index_mask_sums", "total_lengths", "round_number", "rollout_log_probs",
    "rollout_routed_experts", "metadata", "multimodal_train_inputs", "teacher_log_probs", "weight_versions",
)
RolloutBatch = dict
SFTBatch = dict


class MultimodalTypes:
    IMAGE = "image"
    VIDEO = "video"
    AUDIO = "audio"

    @classmethod
    def all(cls):
        return (cls.IMAGE, cls.VIDEO, cls.AUDIO)
