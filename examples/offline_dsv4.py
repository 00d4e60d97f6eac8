"""One chat prompt through the offline API on 8 GPUs (examples/offline_dsv4.py of the reference).

    python examples/offline_dsv4.py /models/DeepSeek-V4-Flash
    python examples/offline_dsv4.py /path/to/small-checkpoint --tp 2 --device cpu --page-size 16 --num-pages 64
"""
import argparse

from minisgl.core import SamplingParams
from minisgl.distributed import launch_tensor_parallel
from minisgl.llm import LLM


def main(model_path: str, prompt: str, max_tokens: int, engine_kw: dict):
    llm = LLM(model_path, **engine_kw)
    messages = [{"role": "user", "content": prompt}]
    out = llm.generate([messages], SamplingParams(temperature=0.6, max_tokens=max_tokens), reasoning_effort=None)[0]
    if llm.tp.is_primary():
        print(out.text)
    llm.shutdown()


def cli(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("model")
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--prompt", default="Explain sliding-window attention in two sentences.")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--device", default="cuda", help="cpu runs the PyTorch oracle (small checkpoints only)")
    ap.add_argument("--page-size", type=int, default=0)
    ap.add_argument("--num-pages", type=int, default=0)
    a = ap.parse_args(argv)
    kw = {"device": a.device}
    if a.device == "cuda":
        kw["recipe"] = "long_context_m8"
    if a.page_size:
        kw["page_size"] = a.page_size
    if a.num_pages:
        kw["num_page_override"] = a.num_pages
    launch_tensor_parallel(a.tp, main, (a.model, a.prompt, a.max_tokens, kw))


if __name__ == "__main__":
    cli()
