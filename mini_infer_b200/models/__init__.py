"""Architectures this engine builds.  Importing the package registers them by name."""

from . import bogetar, nipapel, qwen2_moe, tofinex, vizalix  # noqa: F401
