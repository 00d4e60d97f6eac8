from .detokenize import DetokenizeManager  # noqa: F401
from .tokenize import TokenizeManager, load_dsv4_chat_formatter  # noqa: F401
