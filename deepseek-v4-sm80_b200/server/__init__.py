from .args import ServerArgs, parse_args  # noqa: F401
