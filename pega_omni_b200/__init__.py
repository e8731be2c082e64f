"""B200-native codec-frame token loop behind the reference's model-shell API.

The compute lives in ``libomni_b200.so`` (hand-written CUDA for sm_100a behind a
C ABI, see ``include/omni_b200.h``); this package is the thin Python mirror of
the reference's ``Model`` (crates/omni-qwen3-tts/src/model.rs) used by the
tests and the benchmark. There is no CPU or library fallback: importing
:mod:`pega_omni_b200.lib` raises if the shared library has not been built.
"""
from .config import StackConfig, TalkerConfig, Generation, presets  # noqa: F401

__all__ = ["StackConfig", "TalkerConfig", "Generation", "presets"]
