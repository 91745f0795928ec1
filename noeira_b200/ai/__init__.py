from .chat import ChatClient, parse_sse  # noqa: F401
