"""HuggingFace helpers: tokenizer (with a separately shipped ``chat_template.json``), config loading that falls back
to the raw ``config.json`` when transformers does not know ``deepseek_v4``, and weight folder resolution
(python/minisgl/utils/hf.py:17-64 of the reference)."""
from __future__ import annotations

import functools
import json
import os


def load_tokenizer(model_path: str):
    from transformers import AutoTokenizer
    from transformers.utils import logging as hf_logging

    # transformers does not know the deepseek_v4 model type and says so at length while it only loads the tokenizer
    level = hf_logging.get_verbosity()
    hf_logging.set_verbosity_error()
    try:
        tok = AutoTokenizer.from_pretrained(model_path, trust_remote_code=False)
    finally:
        hf_logging.set_verbosity(level)
    tmpl = os.path.join(model_path, "chat_template.json")
    if getattr(tok, "chat_template", None) is None and os.path.exists(tmpl):
        data = json.load(open(tmpl))
        tok.chat_template = data.get("chat_template", data) if isinstance(data, dict) else data
    return tok


@functools.lru_cache(maxsize=8)
def cached_load_hf_config(model_path: str):
    """Returns the config as a dict-like object usable by ModelConfig.from_hf."""
    cfg_file = os.path.join(model_path, "config.json")
    if os.path.exists(cfg_file):
        return json.load(open(cfg_file))
    from transformers import AutoConfig

    return AutoConfig.from_pretrained(model_path)


def download_hf_weight(model_path: str) -> str:
    if os.path.isdir(model_path):
        return model_path
    from huggingface_hub import snapshot_download

    return snapshot_download(model_path, allow_patterns=["*.safetensors", "*.json"])
