from .backend import AbortBackendMsg, BatchBackendMsg, ExitMsg, UserMsg  # noqa: F401
from .frontend import BatchFrontendMsg, UserReply  # noqa: F401
from .tokenizer import AbortMsg, BatchTokenizerMsg, DetokenizeMsg, TokenizeMsg  # noqa: F401
from .utils import decode, encode, pack, unpack  # noqa: F401
