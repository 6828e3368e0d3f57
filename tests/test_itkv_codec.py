"""The strict ITKV decoder through its host-only entry point (itk_itkv_check, no device): both format versions are
accepted, and every forgery the reference's own tests try (crates/itak-kv/src/snapshot.rs:709-813) - plus their
version-2 forms - is refused by name.  The oracle's encoder supplies the version-1 bytes, a hand-written encoder
(tests/kvparity.py) the version-2 bytes."""
import struct

import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaComputeError, _lib
from itak_torch_rebuild_b200.prefix_store import check_itkv
from kvparity import typed_itkv_bytes
from oracle import oracle as orc

WINDOW, HKV, D = [4, 0], 2, 3


def snapshot(tokens=6, fingerprint="model-a"):
    cache = orc.KvCache([orc.LayerKind.Windowed(4), orc.GLOBAL], HKV, D)
    rng = np.random.default_rng(tokens)
    for position in range(tokens):
        for layer in range(2):
            cache.append(layer, rng.standard_normal(HKV * D).astype(np.float32),
                         rng.standard_normal(HKV * D).astype(np.float32), position)
    return orc.KvSnapshot.capture(cache, fingerprint)


def resum(data):
    return bytes(data[:-8]) + struct.pack("<Q", orc.checksum(bytes(data[:-8])))


def refusal(data):
    with pytest.raises(CudaComputeError) as e:
        check_itkv(bytes(data))
    return e.value


def test_both_versions_decode():
    snap = snapshot()
    assert check_itkv(snap.to_bytes()) == (1, 6, 4)
    assert check_itkv(typed_itkv_bytes(snap, "model-a", HKV, D, WINDOW, half=True)) == (2, 6, 2)
    assert check_itkv(typed_itkv_bytes(snap, "model-a", HKV, D, WINDOW, half=False)) == (2, 6, 4)


@pytest.mark.parametrize("half", [None, True, False])
def test_forgeries_are_refused_by_name(half):
    snap = snapshot()
    good = snap.to_bytes() if half is None else typed_itkv_bytes(snap, "model-a", HKV, D, WINDOW, half=half)
    flipped = bytearray(good)
    flipped[len(good) - 12] ^= 0x40
    assert refusal(flipped).code == _lib.ERR_CHECKSUM_MISMATCH
    for cut in (0, 3, 8, 11, 20, len(good) // 2, len(good) - 9, len(good) - 1):
        assert refusal(good[:cut]).code in (_lib.ERR_TRUNCATED, _lib.ERR_INCONSISTENT_SNAPSHOT), cut
    bad = bytearray(good)
    bad[0] = ord("X")
    assert refusal(bad).code == _lib.ERR_BAD_MAGIC
    future = bytearray(good)
    future[4] = 9
    assert refusal(future).code == _lib.ERR_UNSUPPORTED_VERSION
    e = refusal(good + b"\0\0")
    assert e.code == _lib.ERR_INCONSISTENT_SNAPSHOT and "trailing" in e.msg
    # a layer count far beyond what the bytes could hold must be refused before anything is allocated
    head = 12 if half is None else 16
    fp_len = struct.unpack_from("<I", good, head - 4)[0]
    at = head + fp_len + 8 + 4 + 4
    many = bytearray(good)
    many[at:at + 4] = struct.pack("<I", 0xFFFFFFFF)
    e = refusal(resum(many))
    assert e.code == _lib.ERR_INCONSISTENT_SNAPSHOT and "layers" in e.msg
    # reserved bytes, an unknown layer kind, a zero window on a windowed layer
    first_layer = at + 4
    for offset, value, word in ((1, 1, "reserved"), (0, 5, "kind"),):
        forged = bytearray(good)
        forged[first_layer + offset] = value
        e = refusal(resum(forged))
        assert e.code == _lib.ERR_INCONSISTENT_SNAPSHOT and word in e.msg
    zero_window = bytearray(good)
    zero_window[first_layer + 4:first_layer + 12] = bytes(8)
    assert refusal(resum(zero_window)).code == _lib.ERR_INCONSISTENT_SNAPSHOT
    # a row count that disagrees with the token count
    rows_at = first_layer + 4 + 8 + 8
    wrong = bytearray(good)
    wrong[rows_at:rows_at + 8] = struct.pack("<Q", 3)
    assert refusal(resum(wrong)).code in (_lib.ERR_INCONSISTENT_SNAPSHOT, _lib.ERR_TRUNCATED)


def test_overflowing_products_are_refused():
    """snapshot.rs:769-813: sizes whose products wrap must not reach an allocation or a copy."""
    for version_fields in (struct.pack("<I", 1), struct.pack("<II", 2, 1), struct.pack("<II", 2, 0)):
        forged = b"ITKV" + version_fields + struct.pack("<I", 1) + b"x"
        forged += struct.pack("<QIII", 1 << 40, 0xFFFFFFFF, 0xFFFFFFFF, 1)
        forged += bytes(4) + struct.pack("<QQQ", 0, 0, 1 << 40)
        forged += struct.pack("<Q", orc.checksum(forged))
        assert refusal(forged).code == _lib.ERR_INCONSISTENT_SNAPSHOT
    unknown = b"ITKV" + struct.pack("<III", 2, 7, 0) + struct.pack("<QIII", 0, 1, 1, 0)
    unknown += struct.pack("<Q", orc.checksum(unknown))
    e = refusal(unknown)
    assert e.code == _lib.ERR_INCONSISTENT_SNAPSHOT and "element type" in e.msg
