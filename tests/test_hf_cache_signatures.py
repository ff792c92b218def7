"""The HF cache keeps the reference's interface: for every public method of the reference's
``CompressedKVCache`` the parameters (names, order, defaults) are a prefix of ours; anything we
add is keyword-only with a default.  Runs where the reference tree is importable (it does not
travel to the GPU box)."""
import inspect
import os
import sys

import pytest

# where the build container keeps the reference tree (overridable); absent elsewhere -> skipped
REF_SRC = os.environ.get("FTQ_REFERENCE_SRC", os.path.join(os.sep, "root", "reference", "src"))


def _load_reference():
    if not os.path.isdir(REF_SRC):
        pytest.skip("reference tree not present")
    sys.path.insert(0, REF_SRC)
    try:
        from fused_turboquant.hf.fused_cache import CompressedKVCache
        return CompressedKVCache
    except Exception as e:  # missing optional dependency of the reference
        pytest.skip(f"reference not importable here: {e}")
    finally:
        sys.path.remove(REF_SRC)


def test_public_methods_match_the_reference():
    ref = _load_reference()
    from fused_turboquant_b200.hf_cache import CompressedKVCache as ours
    names = [n for n, f in vars(ref).items() if callable(f) and (not n.startswith("_") or n == "__init__")]
    assert {"store_compressed_key", "store_compressed_value", "store_compressed_kv",
            "get_compressed_key", "get_compressed_value", "decode_values", "reset",
            "set_layer_quantizer", "set_layer_quantizer_v", "get_layer_quantizer",
            "get_layer_quantizer_v"} <= set(names)
    for n in names:
        assert hasattr(ours, n), f"missing method {n}"
        rp = list(inspect.signature(getattr(ref, n)).parameters.values())
        op = list(inspect.signature(getattr(ours, n)).parameters.values())
        for a, b in zip(rp, op):
            assert (a.name, a.kind, a.default) == (b.name, b.kind, b.default), (n, a, b)
        for extra in op[len(rp):]:
            assert extra.kind in (inspect.Parameter.KEYWORD_ONLY, inspect.Parameter.VAR_KEYWORD,
                                  inspect.Parameter.VAR_POSITIONAL), (n, extra)
            assert extra.kind != inspect.Parameter.KEYWORD_ONLY or extra.default is not inspect.Parameter.empty


def test_base_class_is_the_references():
    ref = _load_reference()
    from fused_turboquant_b200.hf_cache import CompressedKVCache as ours
    assert [b.__name__ for b in ours.__mro__[1:2]] == [b.__name__ for b in ref.__mro__[1:2]]
