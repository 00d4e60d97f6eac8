from .llm import LLM, RequestOutput  # noqa: F401
