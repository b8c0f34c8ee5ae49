"""Architectures this engine builds.  Importing the package registers them by name."""

from . import nipapel, qwen2_moe, tofinex, vizalix  # noqa: F401
