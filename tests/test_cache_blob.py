"""Host-side checks of the prepacked-cache blob format (ruyb200_cache_blob_info needs no device): a blob
written by hand from the documented layout is accepted, and every kind of damage or version skew is refused."""
import struct

import numpy as np
import pytest

import ruy_b200
from ruy_b200 import _abi
from ruy_b200.api import cache_blob_info


def fnv1a(data, h=14695981039346656037):
    for b in data:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def make_blob(width=24, depth=40, dtype=_abi.I8, side=0, zero_point=-3, abi=_abi.ABI_VERSION, fmt=_abi.CACHE_FORMAT_ROWS16,
              packed_depth=None, seed=0):
    """Header (64 bytes, little endian): magic, abi, format, dtype/side/has_sums/0, width, depth, packed depth,
    zero point, four zero bytes, data bytes, sums bytes, FNV-1a over the 56 bytes before the checksum and the payload."""
    pd = (depth + 15) // 16 * 16 if packed_depth is None else packed_depth
    rng = np.random.default_rng(seed)
    data = np.zeros((width, pd), dtype=np.int8)
    data[:, :depth] = rng.integers(-127, 127, size=(width, depth), endpoint=True)
    sums = data.astype(np.int32).sum(axis=1).astype("<i4")
    payload = data.tobytes() + sums.tobytes()
    head = struct.pack("<8sIIBBBBiiii4xQQ", b"RUYB2PCK", abi, fmt, dtype, side, 1, 0, width, depth, pd, zero_point,
                       width * pd, 4 * width)
    assert len(head) == 56
    return head + struct.pack("<Q", fnv1a(payload, fnv1a(head))) + payload


def test_hand_written_blob_is_accepted():
    info = cache_blob_info(make_blob())
    assert info == {"abi_version": _abi.ABI_VERSION, "format": 1, "dtype": _abi.I8, "side": 0, "has_sums": 1, "width": 24,
                    "depth": 40, "packed_depth": 48, "zero_point": -3, "data_bytes": 24 * 48, "sums_bytes": 96}


def test_both_row_lengths_of_deep_8bit_rows_are_accepted():
    """8-bit rows of 256 bytes and more are written padded to whole 128-byte lines; a blob whose rows are padded to 16
    bytes only (the earlier layout) is still taken; any other row length is refused."""
    assert cache_blob_info(make_blob(width=8, depth=300, packed_depth=384))["packed_depth"] == 384
    assert cache_blob_info(make_blob(width=8, depth=300, packed_depth=304))["packed_depth"] == 304
    with pytest.raises(ruy_b200.RuyError) as e:
        cache_blob_info(make_blob(width=8, depth=300, packed_depth=320))
    assert e.value.status == _abi.ERR_INVALID
    # below 256 bytes of depth there is only the 16-byte rounding
    with pytest.raises(ruy_b200.RuyError):
        cache_blob_info(make_blob(width=8, depth=200, packed_depth=256))


@pytest.mark.parametrize("damage", ["magic", "abi", "format", "truncated", "payload", "header_field", "packed_depth", "short"])
def test_damaged_or_foreign_blobs_are_refused(damage):
    blob = bytearray(make_blob())
    if damage == "magic":
        blob[0] ^= 1
    elif damage == "abi":
        blob = bytearray(make_blob(abi=_abi.ABI_VERSION + 1))
    elif damage == "format":
        blob = bytearray(make_blob(fmt=7))
    elif damage == "truncated":
        blob = blob[:-1]
    elif damage == "payload":
        blob[64 + 5] ^= 0x10
    elif damage == "header_field":
        blob[24] ^= 1          # the width, without fixing sizes or checksum
    elif damage == "packed_depth":
        blob = bytearray(make_blob(packed_depth=64))   # self-consistent, but not this library's layout for depth 40
    elif damage == "short":
        blob = blob[:40]
    with pytest.raises(ruy_b200.RuyError) as e:
        cache_blob_info(bytes(blob))
    assert e.value.status == _abi.ERR_INVALID
