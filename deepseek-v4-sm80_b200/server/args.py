"""Command-line arguments of ``python -m minisgl`` -> frozen ``ServerArgs``.

Flag names, aliases and defaults follow the reference (python/minisgl/server/args.py:23-303).  The parser remembers
which options the user passed explicitly, so a recipe fills in only what was left unset.  Shell mode serves one
request at a time.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import sys
from dataclasses import dataclass
from typing import List, Optional, Tuple

from ..dsv4_release import RECIPES
from ..parallel.info import DistributedInfo
from ..scheduler.config import SchedulerConfig
from ..utils.misc import UNSET


@dataclass(frozen=True)
class ServerArgs(SchedulerConfig):
    server_host: str = "127.0.0.1"
    server_port: int = 1919
    num_tokenizer: int = 0
    served_model_name: Optional[str] = None
    silent_output: bool = False
    shell_mode: bool = False

    @property
    def share_tokenizer(self) -> bool:
        return self.num_tokenizer == 0

    @property
    def model_names(self) -> Tuple[str, ...]:
        """Names a request may use for this model: the served name and the full path."""
        names = [self.served_model_name or os.path.basename(os.path.normpath(self.model_path)), self.model_path]
        return tuple(dict.fromkeys(n for n in names if n))

    @property
    def zmq_frontend_addr(self) -> str:
        return f"ipc:///tmp/minisgl_b200_frontend{self._unique_suffix}"

    @property
    def zmq_tokenizer_addr(self) -> str:
        return f"ipc:///tmp/minisgl_b200_tokenizer{self._unique_suffix}"

    @property
    def tokenizer_create_addr(self) -> bool:
        return self.share_tokenizer

    @property
    def backend_create_detokenizer_link(self) -> bool:
        return not self.share_tokenizer

    @property
    def distributed_addr_resolved(self) -> str:
        return self.distributed_addr or f"tcp://127.0.0.1:{self.server_port + 1}"


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="minisgl", description="B200-native DeepSeek-V4 serving engine")
    p.add_argument("--model", "--model-path", dest="model_path", required=True)
    p.add_argument("--served-model-name", default=None)
    p.add_argument("--tp-size", "--tensor-parallel-size", dest="tp_size", type=int, default=1)
    p.add_argument("--max-running-requests", dest="max_running_req", type=int, default=None)
    p.add_argument("--enable-reasoning-sampler-contract", action="store_true")
    p.add_argument("--recipe", choices=sorted(RECIPES), default=None)
    p.add_argument("--context-length", "--max-model-len", dest="context_length", type=int, default=None)
    p.add_argument("--memory-ratio", type=float, default=0.9)
    p.add_argument("--dummy-weight", dest="use_dummy_weight", action="store_true")
    p.add_argument("--disable-pynccl", dest="use_pynccl", action="store_false",
                   help="use torch.distributed collectives instead of the fused NVLink kernels")
    p.add_argument("--moe-mode", choices=["ep", "tp"], default="ep")
    p.add_argument("--host", dest="server_host", default="127.0.0.1")
    p.add_argument("--port", dest="server_port", type=int, default=1919)
    p.add_argument("--cuda-graph-max-bs", "--graph", dest="cuda_graph_max_bs", type=int, default=None)
    p.add_argument("--num-tokenizer", type=int, default=0)
    p.add_argument("--max-prefill-length", "--max-extend-length", dest="max_extend_tokens", type=int, default=8192)
    p.add_argument("--stats-log-interval", type=float, default=10.0)
    p.add_argument("--disable-log-stats", action="store_true")
    p.add_argument("--num-pages", dest="num_page_override", type=int, default=None)
    p.add_argument("--page-size", type=int, default=256)
    p.add_argument("--shell-mode", action="store_true")
    p.add_argument("--device", choices=["cuda", "cpu"], default="cuda",
                   help="cpu runs the PyTorch oracle of every operator: for trying the serving stack without a GPU")
    return p


def _explicit(parser: argparse.ArgumentParser, argv: List[str]) -> frozenset:
    seen = set()
    for action in parser._actions:
        for opt in action.option_strings:
            if any(a == opt or a.startswith(opt + "=") for a in argv):
                seen.add(action.dest)
    return frozenset(seen)


def parse_args(argv: Optional[List[str]] = None, run_shell: bool = False) -> ServerArgs:
    argv = list(sys.argv[1:] if argv is None else argv)
    parser = build_parser()
    ns = parser.parse_args(argv)
    explicit = _explicit(parser, argv)
    if ns.tp_size < 1:
        parser.error("--tp-size must be >= 1")
    if not 0.0 < ns.memory_ratio <= 1.0:
        parser.error("--memory-ratio must be in (0, 1]")
    if ns.page_size != 256 and "page_size" in explicit and ns.page_size % 4:
        parser.error("--page-size must be a multiple of 4")
    shell = bool(ns.shell_mode or run_shell)
    kw = dict(
        model_path=ns.model_path, tp_info=DistributedInfo(0, ns.tp_size),
        max_running_req=ns.max_running_req if ns.max_running_req is not None else UNSET,
        cuda_graph_max_bs=ns.cuda_graph_max_bs if ns.cuda_graph_max_bs is not None else UNSET,
        context_length=ns.context_length if ns.context_length is not None else UNSET,
        recipe=ns.recipe, page_size=ns.page_size, memory_ratio=ns.memory_ratio,
        num_page_override=ns.num_page_override, use_dummy_weight=ns.use_dummy_weight, use_pynccl=ns.use_pynccl,
        moe_mode=ns.moe_mode, enable_reasoning_sampler_contract=ns.enable_reasoning_sampler_contract,
        max_extend_tokens=ns.max_extend_tokens, max_prefill_length=ns.max_extend_tokens,
        stats_log_interval=ns.stats_log_interval, disable_log_stats=ns.disable_log_stats,
        server_host=ns.server_host, server_port=ns.server_port, num_tokenizer=ns.num_tokenizer,
        served_model_name=ns.served_model_name, shell_mode=shell, explicit_fields=explicit, device=ns.device,
        _unique_suffix=f".pid={os.getpid()}",
    )
    if shell:  # an interactive shell serves one request at a time and keeps the log quiet
        kw.update(max_running_req=1, cuda_graph_max_bs=1, silent_output=True)
    args = ServerArgs(**kw)
    return dataclasses.replace(args, distributed_addr=args.distributed_addr_resolved)
