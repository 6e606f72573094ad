"""Per-environment credit-assignment algorithm configuration (names follow the reference's
``configs/algorithm.py``). ``action_loss_type`` says which trainer loss component the
model-sampled tokens feed: ``rl``, ``ce`` or ``ref_kl``."""

from __future__ import annotations

from typing import Annotated, Any, ClassVar, Literal, TypeAlias

from pydantic import Field

from .base import BaseConfig
from .shared import ClientConfig

ActionLossType = Literal["rl", "ce", "ref_kl"]


class FrozenModelConfig(ClientConfig):
    name: str


class SamplingConfig(BaseConfig):
    # "policy": the live, weight-updated policy; or an inline frozen model served elsewhere
    source: Literal["policy"] | FrozenModelConfig = "policy"


class LinearLengthPenaltyConfig(BaseConfig):
    type: Literal["linear"] = "linear"
    num_output_tokens_weight: float = Field(0.25, ge=0, allow_inf_nan=False)
    num_input_tokens_weight: float = Field(0.1, ge=0, allow_inf_nan=False)
    num_turns_weight: float = Field(0.1, ge=0, allow_inf_nan=False)


class EchoRoleConfig(BaseConfig):
    alpha: float = Field(0.1, gt=0)


class EchoRolesConfig(BaseConfig):
    system: EchoRoleConfig | None = None
    user: EchoRoleConfig | None = None
    assistant: EchoRoleConfig | None = None
    tool: EchoRoleConfig | None = None


class EchoFilterConfig(BaseConfig):
    import_path: str
    kwargs: dict[str, Any] = Field(default_factory=dict)


class BaseAlgoConfig(BaseConfig):
    action_loss_type: ClassVar[ActionLossType] = "rl"
    sampling: SamplingConfig = SamplingConfig()


class GRPOAlgoConfig(BaseAlgoConfig):
    type: Literal["grpo"] = "grpo"
    length_penalty: LinearLengthPenaltyConfig | None = None


class EchoAlgoConfig(BaseAlgoConfig):
    type: Literal["echo"] = "echo"
    length_penalty: LinearLengthPenaltyConfig | None = None
    roles: EchoRolesConfig = EchoRolesConfig(tool=EchoRoleConfig())
    filter: EchoFilterConfig | None = None


class MaxRLAlgoConfig(BaseAlgoConfig):
    type: Literal["max_rl"] = "max_rl"


class RAEAlgoConfig(BaseAlgoConfig):
    type: Literal["rae"] = "rae"
    decay: float = Field(0.95, ge=0.0, lt=1.0)


class HierarchicalGRPOAlgoConfig(BaseAlgoConfig):
    type: Literal["hierarchical_grpo"] = "hierarchical_grpo"
    episode_agents: list[str] = Field(min_length=1)


class OPDAlgoConfig(BaseAlgoConfig):
    type: Literal["opd"] = "opd"
    action_loss_type: ClassVar[ActionLossType] = "ref_kl"
    teacher: FrozenModelConfig


class OPSDAlgoConfig(BaseAlgoConfig):
    type: Literal["opsd"] = "opsd"
    action_loss_type: ClassVar[ActionLossType] = "ref_kl"
    demo_key: str = "demonstration"
    template: str = "Here is an example of an expert response:\n<demonstration>\n{demonstration}\n</demonstration>"


class SFTAlgoConfig(BaseAlgoConfig):
    type: Literal["sft"] = "sft"
    action_loss_type: ClassVar[ActionLossType] = "ce"


class DebugAlgoConfig(BaseAlgoConfig):
    type: Literal["debug"] = "debug"
    advantage: float = Field(1.0, allow_inf_nan=False)


AlgoConfig: TypeAlias = Annotated[
    GRPOAlgoConfig | EchoAlgoConfig | MaxRLAlgoConfig | RAEAlgoConfig | HierarchicalGRPOAlgoConfig | OPDAlgoConfig
    | OPSDAlgoConfig | SFTAlgoConfig | DebugAlgoConfig, Field(discriminator="type")]
