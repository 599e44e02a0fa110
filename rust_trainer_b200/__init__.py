"""B200-native frozen-quantised-linear LoRA training path (host-side mirror over a C ABI)."""
from . import adapter, dp, evalgate, objectives, ops, packing, quants, synth  # noqa: F401
from ._lib import RtError, lib  # noqa: F401
from .frozen import Context, Frozen  # noqa: F401
from .linear import Linear  # noqa: F401
from .model import Model, schedule_lr  # noqa: F401
