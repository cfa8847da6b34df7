"""Chat prompt templates: ChatML, Llama-3, DeepSeek, Mistral, Alpaca, Gemma, Raw, with detection
from the architecture / model name and each format's default stop strings.

Reference parity: ChatTemplateParser (oxide-models/src/chat_template.rs:71-124 detect,
:144-274 render). The server always renders ChatML (oxide-server/src/lib.rs:406); the CLI picks
by `--chat-format`.
"""
from __future__ import annotations

from enum import Enum
from typing import Iterable, Mapping


class ChatFormat(Enum):
    CHATML = "chatml"
    LLAMA3 = "llama3"
    DEEPSEEK = "deepseek"
    MISTRAL = "mistral"
    ALPACA = "alpaca"
    GEMMA = "gemma"
    RAW = "raw"


def detect(arch: str = "", name: str = "") -> ChatFormat:
    s = f"{arch} {name}".lower()
    if "deepseek" in s:
        return ChatFormat.DEEPSEEK
    if "gemma" in s:
        return ChatFormat.GEMMA
    if "llama-3" in s or "llama3" in s:
        return ChatFormat.LLAMA3
    if "mistral" in s or "mixtral" in s:
        return ChatFormat.MISTRAL
    if "alpaca" in s:
        return ChatFormat.ALPACA
    if "qwen" in s or "chatml" in s or "hermes" in s or "yi" in s.split():
        return ChatFormat.CHATML
    return ChatFormat.CHATML


def parse_format(s: str, arch: str = "", name: str = "") -> ChatFormat:
    if not s or s == "auto":
        return detect(arch, name)
    return ChatFormat(s.lower())


def stop_strings(fmt: ChatFormat) -> list[str]:
    return {
        ChatFormat.CHATML: ["<|im_end|>", "<|endoftext|>"],
        ChatFormat.LLAMA3: ["<|eot_id|>", "<|end_of_text|>"],
        ChatFormat.DEEPSEEK: ["<｜end▁of▁sentence｜>", "<|im_end|>"],
        ChatFormat.MISTRAL: ["</s>"],
        ChatFormat.ALPACA: ["</s>", "### Instruction:"],
        ChatFormat.GEMMA: ["<end_of_turn>", "<eos>"],
        ChatFormat.RAW: [],
    }[fmt]


def render_chat(messages: Iterable[Mapping[str, str]], fmt: ChatFormat = ChatFormat.CHATML,
                add_generation_prompt: bool = True) -> str:
    msgs = [(m.get("role", "user"), m.get("content", "") or "") for m in messages]
    out = []
    if fmt == ChatFormat.CHATML:
        for role, c in msgs:
            out.append(f"<|im_start|>{role}\n{c}<|im_end|>\n")
        if add_generation_prompt:
            out.append("<|im_start|>assistant\n")
    elif fmt == ChatFormat.LLAMA3:
        out.append("<|begin_of_text|>")
        for role, c in msgs:
            out.append(f"<|start_header_id|>{role}<|end_header_id|>\n\n{c}<|eot_id|>")
        if add_generation_prompt:
            out.append("<|start_header_id|>assistant<|end_header_id|>\n\n")
    elif fmt == ChatFormat.DEEPSEEK:
        for role, c in msgs:
            if role == "system":
                out.append(c)
            elif role == "user":
                out.append(f"<｜User｜>{c}")
            else:
                out.append(f"<｜Assistant｜>{c}<｜end▁of▁sentence｜>")
        if add_generation_prompt:
            out.append("<｜Assistant｜>")
    elif fmt == ChatFormat.MISTRAL:
        system = ""
        for role, c in msgs:
            if role == "system":
                system = c + "\n\n"
            elif role == "user":
                out.append(f"[INST] {system}{c} [/INST]")
                system = ""
            else:
                out.append(f" {c}</s>")
    elif fmt == ChatFormat.ALPACA:
        for role, c in msgs:
            if role == "system":
                out.append(f"{c}\n\n")
            elif role == "user":
                out.append(f"### Instruction:\n{c}\n\n")
            else:
                out.append(f"### Response:\n{c}\n\n")
        if add_generation_prompt:
            out.append("### Response:\n")
    elif fmt == ChatFormat.GEMMA:
        for role, c in msgs:
            r = "model" if role == "assistant" else "user"
            out.append(f"<start_of_turn>{r}\n{c}<end_of_turn>\n")
        if add_generation_prompt:
            out.append("<start_of_turn>model\n")
    else:
        out.append("\n".join(c for _, c in msgs))
    return "".join(out)
