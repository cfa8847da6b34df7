"""Reasoning / tool-call post-processing and the gRPC-style DTOs.

Reference parity: `<think>` splitting and JSON tool-call parsing
(oxide-server/src/reasoning_tools.rs:20-97), serde DTOs of grpc.rs:8-65 (data classes only; the
reference has no gRPC service either).
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any, Optional


def split_reasoning(text: str, open_tag: str = "<think>", close_tag: str = "</think>") -> tuple[str, str]:
    """Returns (reasoning, answer). An unterminated block counts as reasoning only."""
    start = text.find(open_tag)
    if start < 0:
        return "", text
    end = text.find(close_tag, start + len(open_tag))
    if end < 0:
        return text[start + len(open_tag):].strip(), text[:start].strip()
    reasoning = text[start + len(open_tag):end].strip()
    answer = (text[:start] + text[end + len(close_tag):]).strip()
    return reasoning, answer


@dataclass
class ToolCall:
    name: str
    arguments: dict[str, Any] = field(default_factory=dict)
    id: Optional[str] = None


_TOOL_BLOCK = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def parse_tool_calls(text: str) -> list[ToolCall]:
    """Finds tool calls written as <tool_call>{json}</tool_call> or as a bare JSON object / list
    with `name` and `arguments` (or `parameters`) keys."""
    cands = _TOOL_BLOCK.findall(text)
    if not cands:
        t = text.strip()
        if t.startswith("{") or t.startswith("["):
            cands = [t]
    out: list[ToolCall] = []
    for c in cands:
        try:
            obj = json.loads(c)
        except json.JSONDecodeError:
            continue
        for o in obj if isinstance(obj, list) else [obj]:
            if isinstance(o, dict) and "name" in o:
                args = o.get("arguments", o.get("parameters", {}))
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except json.JSONDecodeError:
                        args = {"raw": args}
                out.append(ToolCall(str(o["name"]), args if isinstance(args, dict) else {"value": args}, o.get("id")))
    return out


@dataclass
class GenerateRequestDto:
    model: str = ""
    prompt: str = ""
    max_tokens: int = 64
    temperature: float = 0.7
    top_p: float = 0.9
    stream: bool = False


@dataclass
class GenerateResponseDto:
    text: str = ""
    token_ids: list[int] = field(default_factory=list)
    finish_reason: str = ""
    prompt_tokens: int = 0
    completion_tokens: int = 0


@dataclass
class HealthResponseDto:
    status: str = "SERVING"
    active_slots: int = 0
    max_slots: int = 0
