"""B200-native frozen-quantised-linear LoRA training path (host-side mirror over a C ABI)."""
from . import quants  # noqa: F401
from ._lib import RtError, lib  # noqa: F401
from .frozen import Context, Frozen  # noqa: F401
