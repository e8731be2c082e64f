"""Shapes and sampling constants of a talker checkpoint.

Field names follow the checkpoint JSON the reference reads
(crates/omni-qwen3/src/config.rs:9-22, crates/omni-qwen3-tts/src/config.rs:13-48).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace


@dataclass(frozen=True)
class StackConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6

    @property
    def qkv_width(self) -> int:
        return (self.num_attention_heads + 2 * self.num_key_value_heads) * self.head_dim

    def layer_weight_bytes(self) -> int:
        """bf16 bytes of one layer's four matrices (the per-layer HBM stream of a decode pass)."""
        h, d = self.hidden_size, self.head_dim
        q, kv, i = self.num_attention_heads * d, self.num_key_value_heads * d, self.intermediate_size
        return 2 * ((q + 2 * kv) * h + h * q + 2 * i * h + h * i)

    def kv_bytes_per_token(self) -> int:
        return self.num_hidden_layers * 2 * self.num_key_value_heads * self.head_dim * 2


@dataclass(frozen=True)
class Generation:
    temperature: float = 0.9
    top_k: int = 50
    repetition_penalty: float = 1.05
    subtalker_temperature: float = 0.9
    subtalker_top_k: int = 50
    top_p: float = 1.0           # 1.0 = the reference's behaviour (no nucleus filter)
    sampler: str = "uniforms"    # "uniforms" (reference) or "philox"


@dataclass(frozen=True)
class TalkerConfig:
    talker: StackConfig
    predictor: StackConfig
    text_vocab_size: int
    num_code_groups: int = 16
    tts_pad_token_id: int = 0
    codec_eos_token_id: int = 0
    min_frames: int = 2          # talker.rs:52
    control_tokens: int = 1024   # talker.rs:54
    generation: Generation = field(default_factory=Generation)

    def with_generation(self, **kw) -> "TalkerConfig":
        return replace(self, generation=replace(self.generation, **kw))

    # ---- algorithmic HBM bytes of one decode tick (weights streamed once per pass + KV) ----
    def tick_weight_bytes(self) -> int:
        t, p, g = self.talker, self.predictor, self.num_code_groups
        talker = t.num_hidden_layers * t.layer_weight_bytes() + 2 * t.vocab_size * t.hidden_size
        per_pass = p.num_hidden_layers * p.layer_weight_bytes() + 2 * p.hidden_size * t.hidden_size
        heads = (g - 1) * 2 * p.vocab_size * p.hidden_size
        return talker + (g - 1) * per_pass + heads

    def tick_folded_bytes(self, sessions: int) -> int:
        """What the persistent kernel does NOT stream of tick_weight_bytes(): from the second predictor pass on the input
        projection and the first layer's q|k|v projection are table rows computed at load (one projected row and one
        q|k|v row per session and pass are read instead)."""
        t, p, g = self.talker, self.predictor, self.num_code_groups
        if g <= 2:
            return 0
        qkv = (p.num_attention_heads + 2 * p.num_key_value_heads) * p.head_dim
        per_pass = 2 * (p.hidden_size * t.hidden_size + qkv * p.hidden_size)
        rows = 2 * sessions * (p.hidden_size + qkv)
        return (g - 2) * (per_pass - rows)

    def tick_kv_bytes(self, lens) -> int:
        """KV bytes a tick reads (positions 0..len-1 of every session) plus the row it writes."""
        per = self.talker.kv_bytes_per_token()
        return per * (int(sum(lens)) + len(lens))


def _qwen3_tts_1p7b() -> TalkerConfig:
    # Qwen3-TTS-12Hz-1.7B talker; predictor heads / intermediate as in the public checkpoint
    talker = StackConfig(2048, 6144, 28, 16, 8, 128, 3072)
    predictor = StackConfig(1024, 3072, 5, 16, 8, 128, 2048)
    return TalkerConfig(talker, predictor, text_vocab_size=151936, tts_pad_token_id=151671,
                        codec_eos_token_id=2150)


def _tiny128() -> TalkerConfig:
    # reference-compatible shapes (head_dim 128, 16 groups) small enough for the CPU oracle
    talker = StackConfig(256, 768, 2, 4, 2, 128, 3072)
    predictor = StackConfig(128, 384, 2, 2, 1, 128, 2048)
    return TalkerConfig(talker, predictor, text_vocab_size=4096, tts_pad_token_id=4001, codec_eos_token_id=2150)


def _tiny64() -> TalkerConfig:
    # "tiny Qwen3-style codec talker": head_dim 64, 4 codebooks of 2048, 1-layer hidden-128 predictor
    talker = StackConfig(256, 768, 2, 4, 2, 64, 2048)
    predictor = StackConfig(128, 384, 1, 2, 1, 64, 2048)
    return TalkerConfig(talker, predictor, text_vocab_size=4096, num_code_groups=4, tts_pad_token_id=4001,
                        codec_eos_token_id=1100)


def _mid() -> TalkerConfig:
    # mid-size shapes that exercise split-K and several tiles while staying oracle-friendly
    talker = StackConfig(1024, 3072, 3, 8, 4, 128, 3072)
    predictor = StackConfig(512, 1536, 2, 8, 4, 128, 2048)
    return TalkerConfig(talker, predictor, text_vocab_size=8192, tts_pad_token_id=8001, codec_eos_token_id=2150)


presets = {
    "qwen3-tts-1.7b": _qwen3_tts_1p7b,
    "tiny128": _tiny128,
    "tiny64": _tiny64,
    "mid": _mid,
}
