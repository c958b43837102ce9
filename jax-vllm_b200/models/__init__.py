from . import qwen3  # noqa: F401
