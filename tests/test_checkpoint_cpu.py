"""NVFP4 checkpoint container: the C ABI's writer and reader against the CPU restatement of the reference's
format (src/checkpoint/format/{writer,reader}.rs).  Host-only entries: no GPU needed."""
import os
import struct

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import checkpoint as oracle_ckpt


@pytest.fixture(scope="module")
def pkg():
    return entry.load_package()


def sample_tensors(seed=5):
    rng = np.random.default_rng(seed)
    out = []
    # names in the style of the reference's schema (src/checkpoint/save/topology.rs:14-71); ragged sizes, an empty tensor, and a
    # non-ASCII name (names are UTF-8 with an explicit length)
    for name, length in [("token_embedding", 32000 * 16), ("blocks.0.attn_qkv.weight", 768 * 2304),
                         ("blocks.0.mlp_up.bias", 3072), ("ln_f.weight", 768), ("empty", 0),
                         ("\u00e9tage.\u03b2", 160)]:
        data = rng.integers(0, 256, length // 2, dtype=np.uint8).tobytes()
        scales = rng.integers(0, 256, length // 16, dtype=np.uint8).tobytes()
        gs = float(np.float32(rng.uniform(1e-4, 3.0)))
        out.append((name, length, gs, data, scales))
    return out


def test_writer_bytes_equal_the_reference_layout(pkg, tmp_path):
    tensors = sample_tensors()
    path = str(tmp_path / "model.ckpt")
    w = pkg.CheckpointWriter(path, len(tensors))
    for t in tensors:
        w.write_tensor(*t)
    w.finish()
    blob = open(path, "rb").read()
    assert blob == oracle_ckpt.write_checkpoint(tensors)
    # known answer for the fixed-width fields of the header and of the first tensor
    assert blob[:22] == b"GPT2_NVFP4_CHECKPOINT\n"
    assert struct.unpack_from("<II", blob, 22) == (2, len(tensors))
    assert struct.unpack_from("<IQQQ", blob, 30) == (15, 512000, 256000, 32000)


def test_reader_round_trip_and_oracle_written_file(pkg, tmp_path):
    tensors = sample_tensors(9)
    path = str(tmp_path / "from_oracle.ckpt")
    with open(path, "wb") as f:
        f.write(oracle_ckpt.write_checkpoint(tensors))
    r = pkg.CheckpointReader(path)
    assert r.read_header() == len(tensors)
    for want in tensors:
        got = r.read_tensor()
        assert (got.name, got.len, got.bytes, got.scales) == (want[0], want[1], want[3], want[4])
        assert np.float32(got.global_scale) == np.float32(want[2])
    with pytest.raises(pkg.Nvfp4Error, match="no tensor left"):
        r.read_tensor()
    r.close()
    assert oracle_ckpt.read_checkpoint(open(path, "rb").read()) == [
        (n, l, float(np.float32(g)), b, s) for n, l, g, b, s in tensors]


def test_header_errors_are_the_reference_errors(pkg, tmp_path):
    good = oracle_ckpt.write_checkpoint(sample_tensors()[:1])
    bad_magic = str(tmp_path / "magic.ckpt")
    open(bad_magic, "wb").write(b"GPT2_NVFP4_CHECKPOINT " + good[22:])
    with pytest.raises(pkg.Nvfp4Error, match="invalid GPT2 NVFP4 checkpoint magic"):
        pkg.CheckpointReader(bad_magic)
    with pytest.raises(ValueError, match="invalid GPT2 NVFP4 checkpoint magic"):
        oracle_ckpt.read_checkpoint(open(bad_magic, "rb").read())
    bad_version = str(tmp_path / "version.ckpt")
    open(bad_version, "wb").write(good[:22] + struct.pack("<I", 3) + good[26:])
    with pytest.raises(pkg.Nvfp4Error, match="unsupported checkpoint version"):
        pkg.CheckpointReader(bad_version)
    truncated = str(tmp_path / "short.ckpt")
    open(truncated, "wb").write(good[:-5])
    r = pkg.CheckpointReader(truncated)
    with pytest.raises(pkg.Nvfp4Error, match="truncated"):
        r.read_tensor()
    r.close()
    with pytest.raises(pkg.Nvfp4Error, match="cannot open"):
        pkg.CheckpointReader(str(tmp_path / "absent.ckpt"))


def test_writer_count_is_checked(pkg, tmp_path):
    t = sample_tensors()[2]
    w = pkg.CheckpointWriter(str(tmp_path / "a.ckpt"), 1)
    w.write_tensor(*t)
    with pytest.raises(pkg.Nvfp4Error, match="more tensors"):
        w.write_tensor(*t)
    w.finish()
    w = pkg.CheckpointWriter(str(tmp_path / "b.ckpt"), 2)
    w.write_tensor(*t)
    with pytest.raises(pkg.Nvfp4Error, match="fewer tensors"):
        w.finish()


def test_upload_length_rule(pkg):
    ok = ("w", 64, 1.0, bytes(32), bytes(4))
    oracle_ckpt.validate_for_upload(ok)
    with pytest.raises(ValueError, match="expected 32"):
        oracle_ckpt.validate_for_upload(("w", 64, 1.0, bytes(31), bytes(4)))
    with pytest.raises(ValueError, match="expected 4"):
        oracle_ckpt.validate_for_upload(("w", 64, 1.0, bytes(32), bytes(5)))
