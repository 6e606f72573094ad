"""Model-name -> (tool-call parser, reasoning parser) table for the OpenAI-compatible chat
route of the inference server (reference: src/prime_rl/utils/parsers.py)."""

from __future__ import annotations

import re

_TABLE: list[tuple[str, str | None, str | None]] = [
    (r"qwen3.*coder", "qwen3_coder", None),
    (r"qwen3", "hermes", "qwen3"),
    (r"qwen2\.?5", "hermes", None),
    (r"glm-?4\.?[5-9]|glm-?5", "glm45", "glm45"),
    (r"deepseek-?(v3|r1|v4)", "deepseek_v3", "deepseek_r1"),
    (r"gpt-?oss", "openai", "openai_gptoss"),
    (r"minimax-?m2", "minimax_m2", "minimax_m2_append_think"),
    (r"llama-?3", "llama3_json", None),
    (r"nemotron", "hermes", "nemotron"),
    (r"intellect-?3", "qwen3_coder", "deepseek_r1"),
]


def resolve_parsers(model_name: str) -> tuple[str | None, str | None]:
    """(tool_call_parser, reasoning_parser) for a model name; (None, None) when unknown."""
    name = model_name.lower()
    for pattern, tool, reasoning in _TABLE:
        if re.search(pattern, name):
            return tool, reasoning
    return None, None
