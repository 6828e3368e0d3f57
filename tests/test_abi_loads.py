"""CPU-side checks of the boundary: the shared library loads, exports every entry point the header
declares, shares its refusal codes with the oracle, and refuses bad shapes by name before touching a device."""
import ctypes as C
import os
import re

import pytest

import __graft_entry__ as entry
from itak_torch_rebuild_b200 import _lib
from oracle import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "itak_cuda_compute.h")


@pytest.fixture(scope="module")
def lib():
    entry.build()
    return _lib.load()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(itk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert len(names) >= 25
    raw = C.CDLL(_lib.SO_PATH)
    for name in names:
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "the ctypes table and the header disagree"


def test_static_archive_is_built(lib):
    assert os.path.exists(os.path.join(ROOT, "itak_torch_rebuild_b200", "lib", "libitak_cuda_compute.a"))


def test_refusal_codes_match_the_oracle_table():
    text = open(HEADER).read()
    codes = dict((k, int(v)) for k, v in re.findall(r"ITK_ERR_([A-Z_]+)\s*=\s*(\d+)", text))
    for name, value in codes.items():
        if value >= 100:
            continue
        assert getattr(orc, name) == value, name
        assert getattr(_lib, "ERR_" + name) == value, name


def create(lib, **kw):
    cfg = dict(n_layers=2, q_heads=4, kv_heads=2, head_dim=64, n_slots=1, max_context=128, chunk_cap=8,
               kv_dtype=_lib.KV_F16, device=0)
    cfg.update(kw)
    c = _lib.Config(cfg["n_layers"], None, cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["n_slots"],
                    cfg["max_context"], cfg["chunk_cap"], cfg["kv_dtype"], cfg["device"])
    h = C.c_void_p()
    rc = lib.itk_backend_create(C.byref(c), C.byref(h))
    return rc, lib.itk_last_error(None).decode()


def test_create_refuses_bad_shapes_by_name_without_a_device(lib):
    """crates/attention/src/cache.rs:327-351 order: layers, kv heads, head dim; then divisibility."""
    assert create(lib, n_layers=0) == (_lib.ERR_ZERO_DIMENSION, "layer pattern must be positive, got 0")
    assert create(lib, kv_heads=0) == (_lib.ERR_ZERO_DIMENSION, "num_kv_heads must be positive, got 0")
    assert create(lib, head_dim=0) == (_lib.ERR_ZERO_DIMENSION, "head_dim must be positive, got 0")
    rc, msg = create(lib, q_heads=3)
    assert rc == _lib.ERR_NON_DIVISIBLE_HEADS and msg == "3 query heads do not divide evenly across 2 KV heads"
    rc, msg = create(lib, kv_dtype=7)
    assert rc == _lib.ERR_INVALID_ARGUMENT


def test_product_does_not_reach_into_the_oracle():
    """Nothing shipped may import, link or execute the oracle."""
    pkg = os.path.join(ROOT, "itak_torch_rebuild_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower(), (dirpath, f)
