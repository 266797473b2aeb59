"""The safetensors layout validator without a device: it accepts what the format allows and rejects what the
reference's loader rejects (crates/onnx-interop/src/st_load.rs:128-132 and the safetensors format rules: offsets
contiguous from 0 to the end of the buffer, byte length = shape x dtype width)."""
import ctypes as C
import json

import numpy as np
import pytest

from fandhe_ai_b200._lib import BackendError, check, lib
from fandhe_ai_b200.decoder import write_safetensors


def validate(blob: bytes) -> int:
    n = C.c_uint64()
    buf = (C.c_uint8 * max(len(blob), 1)).from_buffer_copy(blob or b"\0")
    check(lib().b200_safetensors_validate(buf, len(blob), C.byref(n)))
    return int(n.value)


def blob_of(header: dict, data: bytes, pad: bool = True) -> bytes:
    text = json.dumps(header).encode()
    if pad:
        text += b" " * (-len(text) % 8)
    return len(text).to_bytes(8, "little") + text + data


def test_a_written_file_validates(tmp_path):
    p = tmp_path / "w.safetensors"
    write_safetensors(p, {"a.qweight": np.arange(12, dtype=np.int8).reshape(3, 4), "a.scale": np.ones(3, np.float32),
                          "b.weight": np.zeros((2, 5), np.float32), "flag": np.array([True, False])})
    assert validate(p.read_bytes()) == 4
    assert validate(blob_of({}, b"")) == 0
    assert validate(blob_of({"__metadata__": {"format": "pt", "note": "é\"x\\"}}, b"")) == 0


@pytest.mark.parametrize("why,blob", [
    ("short file", b"\x01\x00\x00"),
    ("header longer than file", (1000).to_bytes(8, "little") + b"{}"),
    ("header over 100 MB", (200_000_000).to_bytes(8, "little") + b"{}"),
    ("not json", blob_of({}, b"").replace(b"{}", b"[]")),
    ("hole", blob_of({"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8)),
    ("overlap", blob_of({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                         "b": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8)),
    ("length mismatch", blob_of({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)),
    ("trailing data", blob_of({"a": {"dtype": "I8", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 5)),
    ("unknown dtype", blob_of({"a": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4)),
    ("missing field", blob_of({"a": {"dtype": "I8", "shape": [4]}}, b"\0" * 4)),
    ("negative", blob_of({"a": {"dtype": "I8", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4).replace(b"[4]", b"[-4]")),
    ("duplicate", (lambda t: len(t).to_bytes(8, "little") + t + b"\0" * 8)(
        b'{"a":{"dtype":"I8","shape":[4],"data_offsets":[0,4]},"a":{"dtype":"I8","shape":[4],"data_offsets":[4,8]}}')),
])
def test_broken_files_are_rejected(why, blob):
    with pytest.raises(BackendError) as e:
        validate(blob)
    assert e.value.kind == "InvalidArgument", why
    assert "safetensors" in e.value.message
