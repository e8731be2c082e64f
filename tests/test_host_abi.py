"""The C ABI as shipped: the library loads on a machine without a GPU, exports every symbol the headers
declare, and refuses to create a model when no CUDA device is usable (there is no CPU path)."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names |= set(re.findall(r"\b(omni_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol(built_lib):
    from pega_omni_b200 import lib
    declared = declared_symbols()
    assert len(declared) >= 25
    for name in declared:
        assert hasattr(built_lib, name), f"{name} is declared in include/ but not exported"
    assert declared == set(lib.SYMBOLS), "python binding and headers disagree"


def test_bucket_matches_reference_table(built_lib):
    # BUCKETS of crates/omni-kern/src/lib.rs:31
    buckets = [1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128]
    for n in range(1, 129):
        assert built_lib.omni_bucket(n) == next(b for b in buckets if b >= n)
    assert built_lib.omni_bucket(129) == 192 and built_lib.omni_bucket(256) == 256


def test_no_cpu_fallback_without_a_device(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from pega_omni_b200.config import presets
    from pega_omni_b200.model import Limits, Model, OmniError
    from pega_omni_b200.synthetic import random_checkpoint
    cfg = presets["tiny128"]()
    with pytest.raises(OmniError) as e:
        Model.load(0, random_checkpoint(cfg), cfg, Limits(max_batch=2, max_tokens=64, kv_gib=0.001))
    assert e.value.status == -2  # OMNI_ERR_CUDA


def test_struct_layouts_match_header(built_lib):
    from pega_omni_b200 import lib
    assert C.sizeof(lib.Draw) == 128 and C.sizeof(lib.StackCfg) == 36
    assert C.sizeof(lib.Tensor) == 64
    assert C.sizeof(lib.DuplexCfg) == 92 and C.sizeof(lib.DuplexStep) == 112 and C.sizeof(lib.HiggsDelay) == 12
