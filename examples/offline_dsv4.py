"""One chat prompt through the offline API on 8 GPUs (examples/offline_dsv4.py of the reference).

    python examples/offline_dsv4.py /models/DeepSeek-V4-Flash
"""
import sys

from minisgl.core import SamplingParams
from minisgl.distributed import launch_tensor_parallel
from minisgl.llm import LLM


def main(model_path: str):
    llm = LLM(model_path, recipe="long_context_m8")
    messages = [{"role": "user", "content": "Explain sliding-window attention in two sentences."}]
    out = llm.generate([messages], SamplingParams(temperature=0.6, max_tokens=256), reasoning_effort=None)[0]
    if llm.tp.is_primary():
        print(out.text)
    llm.shutdown()


if __name__ == "__main__":
    launch_tensor_parallel(8, main, (sys.argv[1],))
