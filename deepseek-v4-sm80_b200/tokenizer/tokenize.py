"""Prompt encoding.  Chat requests go through the model's own formatter when the checkpoint ships one
(``<model>/encoding/encoding_dsv4.py`` exposing ``encode_messages(messages, thinking_mode, reasoning_effort)``),
otherwise through the HuggingFace chat template (python/minisgl/tokenizer/tokenize.py:12-66 of the reference)."""
from __future__ import annotations

import importlib.util
from pathlib import Path
from typing import Any, Callable, List, Optional

import torch


def load_dsv4_chat_formatter(model_path: str) -> Optional[Callable[[list, Optional[str]], str]]:
    path = Path(model_path) / "encoding" / "encoding_dsv4.py"
    if not path.is_file():
        return None
    spec = importlib.util.spec_from_file_location("minisgl_dsv4_encoding", path)
    if spec is None or spec.loader is None:
        raise RuntimeError(f"failed to load the DeepSeek V4 chat encoding from {path}")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)

    def fmt(messages: list, reasoning_effort: Optional[str]) -> str:
        mode = "thinking" if reasoning_effort is not None else "chat"
        return module.encode_messages(messages, thinking_mode=mode, reasoning_effort=reasoning_effort)

    return fmt


class TokenizeManager:
    def __init__(self, tokenizer, model_path: Optional[str] = None, formatter=None):
        self.tokenizer = tokenizer
        self.formatter = formatter if formatter is not None else (
            load_dsv4_chat_formatter(model_path) if model_path else None)

    def render(self, text: Any, reasoning_effort: Optional[str]) -> str:
        if not isinstance(text, list):
            return text
        if self.formatter is not None:
            return self.formatter(text, reasoning_effort)
        if reasoning_effort is not None:
            raise ValueError("reasoning_effort requires the DeepSeek V4 chat formatter")
        return self.tokenizer.apply_chat_template(text, tokenize=False, add_generation_prompt=True)

    def encode_messages(self, text: Any, reasoning_effort: Optional[str] = None) -> torch.Tensor:
        ids = self.tokenizer.encode(self.render(text, reasoning_effort))
        return torch.tensor(list(ids), dtype=torch.int32)

    def tokenize(self, msgs: List[Any]) -> List[torch.Tensor]:
        return [self.encode_messages(m.text, m.reasoning_effort) for m in msgs]
