"""Credit assignment. An algorithm scores a completed *group* of rollouts of one task
(``score_group``) and turns each rollout into training samples with per-token streams:
``advantages`` and the component weights ``rl_weights`` / ``ce_weights`` / ``ref_kl_weights``
(reference: src/prime_rl/orchestrator/algo/*.py, routing.py).

grpo               advantage = reward - group mean (optional linear length penalty)
max_rl             (r - mean) / mean: low-pass-rate tasks get ~1/p weight
rae                reward minus a per-agent exponential-moving-average baseline
hierarchical_grpo  group baseline within each agent role of multi-agent episodes
echo               GRPO on action tokens + weighted cross-entropy on observation tokens by role
opd / opsd         on-policy (self-)distillation: reverse KL to teacher logprobs (``ref_kl``)
sft                cross-entropy on the sampled tokens
debug              constant advantage
"""

from __future__ import annotations

from collections import defaultdict

from ...transports.batch.types import RoutedExperts, SamplingMask, TrainingSample
from ..types import Rollout


class Algorithm:
    action_loss_type = "rl"

    def __init__(self, config, clients=None):
        self.config, self.clients = config, clients

    async def finalize_episode(self, rollout: Rollout) -> None:
        return

    async def score_group(self, group: list[Rollout]) -> None:
        raise NotImplementedError

    def observation_weights(self, rollout: Rollout, n_tokens: int) -> list[float] | None:
        return None

    # ------------------------------------------------------------------ samples
    def to_samples(self, rollout: Rollout) -> list[TrainingSample]:
        """One sample per rollout: the last turn's prompt + completion covers the whole chain;
        tokens sampled in earlier turns are trainable too (mask true), environment tokens not."""
        last = rollout.turns[-1]
        tokens = list(last.prompt_ids) + list(last.completion_ids)
        n = len(tokens)
        mask, logprobs, temps = [False] * n, [0.0] * n, [1.0] * n
        for t in rollout.turns:
            s = len(t.prompt_ids)
            for i, lp in enumerate(t.completion_logprobs):
                mask[s + i], logprobs[s + i] = True, float(lp)
            for i in range(s, min(n, s + len(t.completion_ids))):
                temps[i] = t.temperature if t.temperature > 0 else 1.0
        adv = rollout.advantage if rollout.advantage is not None else 0.0
        sample = TrainingSample(token_ids=tokens, mask=mask, logprobs=logprobs, temperatures=temps,
                                env_name=rollout.env_name, trace_id=rollout.trace_id, branch_index=0)
        kind = self.action_loss_type
        if kind == "rl":
            sample.advantages = [adv if m else 0.0 for m in mask]
        elif kind == "ce":
            sample.ce_weights = [1.0 if m else 0.0 for m in mask]
            sample.rl_weights = [0.0] * n
            sample.advantages = [0.0] * n
        elif kind == "ref_kl":
            ref = rollout.info.get("ref_logprobs")
            if ref is None:
                raise ValueError(f"{type(self).__name__} needs teacher logprobs on the rollout")
            sample.ref_logprobs = [float(x) for x in ref]
            sample.ref_kl_weights = [1.0 if m else 0.0 for m in mask]
            sample.rl_weights = [0.0] * n
            sample.advantages = [0.0] * n
        obs = self.observation_weights(rollout, n)
        if obs is not None:
            sample.ce_weights = obs
        if last.mm is not None:
            import numpy as np

            from ...transports.batch.types import EncodedTensor

            px = np.ascontiguousarray(np.asarray(last.mm["pixel_values"], dtype=np.float32))
            grid = np.ascontiguousarray(np.asarray(last.mm["image_grid_thw"], dtype=np.int64))
            sample.mm_kwargs = {"pixel_values": EncodedTensor("float32", list(px.shape), px.tobytes()),
                                "image_grid_thw": EncodedTensor("int64", list(grid.shape), grid.tobytes())}
            img = last.mm.get("image_token_id")
            sample.mm_token_type_ids = [1 if (img is not None and t == img) else 0 for t in tokens]
        if len(rollout.turns) == 1 and last.routed_experts is not None:
            import numpy as np

            arr = np.asarray(last.routed_experts)
            pad = np.zeros((len(last.prompt_ids),) + arr.shape[1:], dtype=arr.dtype)
            full = np.concatenate([pad, arr], 0)[:n]
            sample.routed_experts = RoutedExperts(data=full.tobytes(), shape=list(full.shape), dtype=str(full.dtype))
        if len(rollout.turns) == 1 and last.sampling_mask is not None:
            import numpy as np

            ids, counts = last.sampling_mask
            full_counts = np.concatenate([np.zeros(len(last.prompt_ids), np.int32), np.asarray(counts, np.int32)])[:n]
            sample.sampling_mask = SamplingMask(ids=np.asarray(ids, np.int32).tobytes(), counts=full_counts.tobytes())
        return [sample]


def _mean(xs):
    return sum(xs) / max(1, len(xs))


class GRPO(Algorithm):
    async def score_group(self, group):
        rewards = [r.reward for r in group]
        lp = getattr(self.config, "length_penalty", None)
        if lp is not None:
            out = [float(r.num_output_tokens) for r in group]
            inp = [float(r.num_total_tokens - r.num_output_tokens) for r in group]
            turns = [float(r.num_turns) for r in group]
            mo, mi, mt = max(max(out), 1.0), max(max(inp), 1.0), max(max(turns), 1.0)
            mean_r = _mean(rewards)
            rewards = [r - mean_r * (lp.num_output_tokens_weight * o / mo + lp.num_input_tokens_weight * i / mi
                                     + lp.num_turns_weight * t / mt)
                       for r, o, i, t in zip(rewards, out, inp, turns)]
        base = _mean(rewards)
        for r, rew in zip(group, rewards):
            r.advantage = rew - base


class MaxRL(Algorithm):
    async def score_group(self, group):
        mu = _mean([r.reward for r in group])
        for r in group:
            r.advantage = (r.reward - mu) / mu if mu > 1e-8 else 0.0


class RAE(Algorithm):
    def __init__(self, config, clients=None):
        super().__init__(config, clients)
        self.baselines: dict[str, float] = {}

    async def score_group(self, group):
        d = self.config.decay
        for r in group:
            key = f"{r.env_name}/{r.agent or 'agent'}"
            b = self.baselines.get(key, r.reward)
            r.advantage = r.reward - b
            self.baselines[key] = d * b + (1 - d) * r.reward

    def state_dict(self):
        return {"baselines": dict(self.baselines)}

    def load_state_dict(self, sd):
        self.baselines = dict(sd.get("baselines", {}))


class HierarchicalGRPO(Algorithm):
    async def score_group(self, group):
        by_agent = defaultdict(list)
        for r in group:
            by_agent[r.agent if r.agent in self.config.episode_agents else "_other"].append(r)
        for members in by_agent.values():
            base = _mean([r.reward for r in members])
            for r in members:
                r.advantage = r.reward - base


class Echo(GRPO):
    """GRPO plus weighted cross-entropy on observation tokens of the configured roles."""

    def observation_weights(self, rollout, n_tokens):
        roles = self.config.roles
        w = [0.0] * n_tokens
        hit = False
        for t in rollout.turns:
            for role, s, e in t.role_spans:
                rc = getattr(roles, role, None)
                if rc is not None:
                    for i in range(s, min(e, n_tokens)):
                        w[i] = rc.alpha
                        hit = True
        return w if hit else None


class OPD(Algorithm):
    action_loss_type = "ref_kl"

    async def finalize_episode(self, rollout):
        if "ref_logprobs" in rollout.info or self.clients is None:
            return
        last = rollout.turns[-1]
        tokens = list(last.prompt_ids) + list(last.completion_ids)
        teacher = self.clients.teacher(self.config.teacher) if hasattr(self.clients, "teacher") else self.clients
        rollout.info["ref_logprobs"] = await teacher.prompt_logprobs(tokens)

    async def score_group(self, group):
        for r in group:
            r.advantage = 0.0


class OPSD(OPD):
    """Self-distillation: the teacher is the policy itself, conditioned on a demonstration hint."""

    async def finalize_episode(self, rollout):
        if "ref_logprobs" in rollout.info or self.clients is None:
            return
        last = rollout.turns[-1]
        demo = rollout.info.get(self.config.demo_key)
        hint = list(demo) if isinstance(demo, (list, tuple)) else []
        tokens = hint + list(last.prompt_ids) + list(last.completion_ids)
        lps = await self.clients.prompt_logprobs(tokens)
        rollout.info["ref_logprobs"] = lps[len(hint):]


class SFT(Algorithm):
    action_loss_type = "ce"

    async def score_group(self, group):
        for r in group:
            r.advantage = 0.0


class Debug(Algorithm):
    async def score_group(self, group):
        for r in group:
            r.advantage = self.config.advantage


ALGORITHMS = {"grpo": GRPO, "max_rl": MaxRL, "rae": RAE, "hierarchical_grpo": HierarchicalGRPO, "echo": Echo,
              "opd": OPD, "opsd": OPSD, "sft": SFT, "debug": Debug}


def setup_algorithm(config, clients=None) -> Algorithm:
    return ALGORITHMS[config.type](config, clients)
