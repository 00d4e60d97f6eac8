"""B200-native serving engine for the DeepSeek-V4-Flash architecture.

Public surface (same names as the reference package, python/minisgl/):
``python -m minisgl`` (OpenAI-compatible server), ``python -m minisgl.shell``,
``minisgl.llm.LLM``, ``minisgl.distributed.launch_tensor_parallel``,
``minisgl.core.SamplingParams``.
"""
__version__ = "0.1.0+dsv4.b200"
