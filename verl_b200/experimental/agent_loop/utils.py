"""Small helpers of the agent loops.

* ``resolve_config_path`` / ``load_agent_loop_configs``: user-defined agent loops are declared in a YAML file
  (``rollout.agent.agent_loop_config_path``), one entry per loop: ``name``, ``_target_`` (dotted path of the class) and any
  further keys, which are passed to the class as keyword arguments. Worker processes may start in another directory than the
  driver, so a relative path is looked for in the working directory, then beside the package (a source checkout), then
  inside it; it must stay inside the directory it is resolved against.
* gpt-oss tool turns: that model's chat template can only render a tool result next to the assistant message that asked for
  it, so a tool turn rendered on its own is written by hand in the model's channel format.

Parity target: ``verl/experimental/agent_loop/utils.py`` (``resolve_config_path`` :19, gpt-oss helpers :78-108) and the
registry loading in ``verl/experimental/agent_loop/agent_loop.py:500-507``.
"""

from __future__ import annotations

import importlib
import os
from typing import Any

__all__ = ["resolve_config_path", "load_agent_loop_configs", "format_gpt_oss_tool_response_manually",
           "add_generation_prompt_for_gpt_oss", "build_gpt_oss_tool_response_text"]


def _under(root: str, rel: str):
    root = os.path.abspath(root)
    p = os.path.abspath(os.path.join(root, rel))
    return p if (p == root or p.startswith(root + os.sep)) and os.path.exists(p) else None


def resolve_config_path(config_path: str) -> str:
    if os.path.isabs(config_path):
        return config_path
    pkg = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # the package directory
    for root in (os.getcwd(), os.path.dirname(pkg), pkg):
        hit = _under(root, config_path)
        if hit:
            return hit
    raise FileNotFoundError(f"Agent loop configuration file not found: {config_path}. Tried the current directory, the "
                            f"project root and the package directory.")


def load_agent_loop_configs(config_path: str) -> dict[str, tuple[type, dict]]:
    """``name -> (class, extra keyword arguments)`` for every entry of the file."""
    import yaml

    with open(resolve_config_path(config_path)) as f:
        entries = yaml.safe_load(f) or []
    out = {}
    for e in entries:
        e = dict(e)
        name, target = e.pop("name"), e.pop("_target_")
        mod, _, cls = str(target).rpartition(".")
        out[str(name)] = (getattr(importlib.import_module(mod), cls), e)
    return out


def format_gpt_oss_tool_response_manually(tool_response: str, tool_call_name: str) -> str:
    return f"<|start|>functions.{tool_call_name} to=assistant<|channel|>commentary<|message|>{tool_response}<|end|>"


def add_generation_prompt_for_gpt_oss(message_content: str) -> str:
    return message_content + "<|start|>assistant"


def build_gpt_oss_tool_response_text(messages: list[dict[str, Any]], tool_call_names: list[str]) -> str:
    """All tool results of one turn in call order, followed by the generation prompt."""
    if len(messages) != len(tool_call_names):
        raise ValueError(f"{len(messages)} tool messages for {len(tool_call_names)} tool calls")
    return add_generation_prompt_for_gpt_oss("".join(format_gpt_oss_tool_response_manually(m["content"], n)
                                                     for m, n in zip(messages, tool_call_names)))
