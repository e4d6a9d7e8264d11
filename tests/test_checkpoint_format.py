"""The checkpoint file layout (documented in host/include/arraydiff/optimize.hh) as the Python reader sees it:
a file assembled by hand parses back to what went in, and damaged files are refused.  No GPU needed."""
import struct

import numpy as np
import pytest

from arraydiff_cuda_b200 import hostlib


def write(path, params, momentum, stats, iteration, manifest, magic=b"ADB2CKPT", version=1):
    with open(path, "wb") as f:
        f.write(magic + struct.pack("<IQQQI", version, len(params), len(stats), iteration, len(manifest)))
        for name, (off, size) in manifest.items():
            f.write(struct.pack("<I", len(name)) + name.encode() + struct.pack("<QQ", off, size))
        f.write(np.asarray(params, "<f4").tobytes() + np.asarray(momentum, "<f4").tobytes() + np.asarray(stats, "<f4").tobytes())


def test_checkpoint_layout_round_trip(tmp_path):
    rng = np.random.default_rng(1)
    p, m, s = rng.standard_normal(37).astype(np.float32), rng.standard_normal(37).astype(np.float32), rng.standard_normal(6).astype(np.float32)
    man = {"conv.kernel": (0, 27), "bn.scale": (27, 5), "bn.shift": (32, 5)}
    write(tmp_path / "a.bin", p, m, s, 123, man)
    ck = hostlib.read_checkpoint(tmp_path / "a.bin")
    assert (ck["version"], ck["param_dim"], ck["stat_dim"], ck["iteration"]) == (1, 37, 6, 123)
    assert ck["manifest"] == man
    assert np.array_equal(ck["params"], p) and np.array_equal(ck["momentum"], m) and np.array_equal(ck["stats"], s)


def test_checkpoint_reader_refuses_damage(tmp_path):
    p = np.zeros(4, np.float32)
    write(tmp_path / "bad_magic.bin", p, p, [], 0, {}, magic=b"NOTACKPT")
    with pytest.raises(AssertionError):
        hostlib.read_checkpoint(tmp_path / "bad_magic.bin")
    write(tmp_path / "ok.bin", p, p, [], 0, {"w": (0, 4)})
    raw = open(tmp_path / "ok.bin", "rb").read()
    open(tmp_path / "short.bin", "wb").write(raw[:-3])
    with pytest.raises((AssertionError, ValueError)):
        hostlib.read_checkpoint(tmp_path / "short.bin")
