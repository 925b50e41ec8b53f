"""B200-native MTP speculative-decode step of the qwen35 hybrid model (host side of the C ABI)."""
from . import binding, configs, replicas, serve, synth_vocab, tp  # noqa: F401
from .binding import Batch, Context, DeviceArray, Model, ModelConfig, QbError, Weight, lib  # noqa: F401
