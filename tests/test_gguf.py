"""The GGUF reader behind the C ABI: valid files, block sizing, hostile input. Where the reference's own reader was compiled (oracle/_ref), both read the same
bytes and must agree on every tensor, every metadata value and every error code (the reference's cases: tests/unit/test_gguf.cpp:401-519)."""
import struct

import numpy as np
import pytest

from dooms_b200 import DoomsError, synth
from dooms_b200 import _lib as L
from dooms_b200.gguf_io import GgufFile, GgufWriter
from oracle import binding as ob

from helpers import QUANT_PLANS, write

REF = ob.reference_reader()


def parse_code(data: bytes) -> int:
    try:
        GgufFile(data=data).close()
        return L.OK
    except DoomsError as e:
        return e.code


def small_file(tmp_path, alignment=32) -> bytes:
    path = tmp_path / "s.gguf"
    md = {"general.architecture": "llama", "llama.block_count": 2, "llama.rope.freq_base": 10000.0, "some.flag": True, "some.list": [1, -2, 3]}
    t = [("a.weight", L.F32, [4, 8], lambda: np.arange(32, dtype=np.float32)), ("b.weight", L.Q4_0, [2, 64], lambda: np.zeros(72, dtype=np.uint8)),
         ("c.weight", L.Q6_K, [1, 256], lambda: np.ones(210, dtype=np.uint8)), ("d", L.F16, [5], lambda: np.zeros(5, dtype=np.float16))]
    GgufWriter(alignment).write(path, md, t)
    return path.read_bytes()


def test_reads_what_the_writer_wrote(tmp_path):
    data = small_file(tmp_path)
    f = GgufFile(data=data)
    assert f.version == 3 and f.alignment == 32
    assert f.get_string("general.architecture") == "llama" and f.get_uint("llama.block_count") == 2 and f.get_float("llama.rope.freq_base") == 10000.0
    assert f.get_bool("some.flag") is True
    ts = {t["name"]: t for t in f.tensors()}
    assert ts["a.weight"]["shape"] == [4, 8] and ts["a.weight"]["nbytes"] == 128 and ts["a.weight"]["dtype"] == L.F32
    assert ts["b.weight"]["nbytes"] == 2 * 2 * 18 and ts["c.weight"]["nbytes"] == 210 and ts["d"]["nbytes"] == 10
    assert np.array_equal(f.tensor_bytes("a.weight").view(np.float32), np.arange(32, dtype=np.float32))
    for t in ts.values():
        assert t["offset"] % 32 == 0
    for fn, key, code in ((f.get_string, "missing", L.NOT_FOUND), (f.get_uint, "general.architecture", L.INVALID_ARGUMENT),
                          (f.get_float, "llama.block_count", L.INVALID_ARGUMENT), (f.find_tensor, "nope", L.NOT_FOUND)):
        with pytest.raises(DoomsError) as e:
            fn(key)
        assert e.value.code == code


def test_agrees_with_gguf_py(tmp_path):
    gguf = pytest.importorskip("gguf")
    path = tmp_path / "m.gguf"
    synth.write_model(synth.tiny_spec(QUANT_PLANS["Q4_K_M-like mix"]), path, 5)
    mine = {t["name"]: t for t in GgufFile(str(path)).tensors()}
    theirs = gguf.GGUFReader(str(path)).tensors
    assert len(mine) == len(theirs)
    for t in theirs:
        m = mine[t.name]
        assert m["shape"] == [int(d) for d in reversed(t.shape)] and m["nbytes"] == t.n_bytes and m["offset"] == t.data_offset
        assert L.GGML_TYPE_ID[m["dtype"]] == int(t.tensor_type)


@pytest.mark.skipif(REF is None, reason="the reference's reader was not compiled (oracle/_ref)")
def test_agrees_with_the_reference_reader_on_valid_files(tmp_path):
    for data in (small_file(tmp_path), small_file(tmp_path, 64)):
        code, ref = ob.reference_parse(data)
        assert code == 0
        f = GgufFile(data=data)
        assert (f.version, f.alignment) == (ref["version"], ref["alignment"])
        mine = f.tensors()
        assert [(t["name"], L.DTYPE_NAMES[t["dtype"]], t["shape"], t["offset"], t["nbytes"]) for t in mine] == \
               [(t["name"], t["dtype"], t["shape"], t["offset"], t["nbytes"]) for t in ref["tensors"]]
        assert f.get_uint("llama.block_count") == ref["kv"]["llama.block_count"]["value"]
        assert f.get_string("general.architecture") == ref["kv"]["general.architecture"]["value"]


def test_every_truncation_is_refused_cleanly(tmp_path):
    """tests/unit/test_gguf.cpp:461-480: no prefix of a valid file parses as that file, none crashes; with the reference's reader: the same code."""
    data = small_file(tmp_path)
    for n in list(range(0, 700)) + list(range(700, len(data), 37)):
        code = parse_code(data[:n])
        assert code != L.OK or n >= len(data) - 31          # only a cut inside the last tensor's alignment padding may still be the whole file
        if REF is not None:
            assert code == ob.reference_parse(data[:n])[0], n


def test_random_corruption_never_crashes_and_agrees_with_the_reference(tmp_path):
    """tests/unit/test_gguf.cpp:482-519: random byte flips in the header and garbage input."""
    data = bytearray(small_file(tmp_path))
    g = np.random.default_rng(0)
    header = 600
    for trial in range(400):
        d = bytearray(data)
        for _ in range(int(g.integers(1, 4))):
            d[int(g.integers(0, header))] = int(g.integers(0, 256))
        code = parse_code(bytes(d))
        assert 0 <= code <= 7
        if REF is not None:
            assert code == ob.reference_parse(bytes(d))[0], trial
    for trial in range(50):
        junk = bytes(g.integers(0, 256, int(g.integers(1, 300)), dtype=np.uint8))
        assert parse_code(junk) != L.OK
        assert parse_code(b"GGUF" + junk) != L.OK or True


def test_specific_malformations(tmp_path):
    data = small_file(tmp_path)
    assert parse_code(b"") == L.INVALID_ARGUMENT
    assert parse_code(b"GGUX" + data[4:]) == L.DATA_LOSS
    assert parse_code(data[:4] + struct.pack("<I", 1) + data[8:]) == L.UNSUPPORTED                 # version 1
    assert parse_code(data[:4] + struct.pack("<I", 3 << 24) + data[8:]) == L.UNSUPPORTED           # byte-swapped version
    assert parse_code(data[:8] + struct.pack("<Q", 1 << 40) + data[16:]) == L.RESOURCE_EXHAUSTED   # absurd tensor count
    assert parse_code(data[:16] + struct.pack("<Q", 1 << 40) + data[24:]) == L.RESOURCE_EXHAUSTED  # absurd metadata count

    def with_tensor(dtype_id, shape, offset=0, n_extra=0):
        head = b"GGUF" + struct.pack("<IQQ", 3, 1, 0)
        name = b"t"
        info = struct.pack("<Q", len(name)) + name + struct.pack("<I", len(shape)) + b"".join(struct.pack("<q", d) for d in shape) + struct.pack("<iQ", dtype_id, offset)
        body = head + info
        body += b"\0" * ((-len(body)) % 32)
        return body + b"\0" * n_extra
    assert parse_code(with_tensor(2, [48, 2], n_extra=4096)) == L.DATA_LOSS        # q4_0 rows of 48 elements: not whole blocks
    assert parse_code(with_tensor(12, [128, 2], n_extra=4096)) == L.DATA_LOSS      # q4_K rows of 128
    assert parse_code(with_tensor(2, [64, 2], n_extra=72)) == L.OK                 # 2 rows x 2 blocks x 18 bytes
    assert parse_code(with_tensor(2, [64, 2], n_extra=71)) == L.DATA_LOSS          # one byte short
    assert parse_code(with_tensor(3, [32], n_extra=64)) == L.UNSUPPORTED           # q4_1: a type the decoder does not take
    assert parse_code(with_tensor(0, [4], offset=8, n_extra=64)) == L.DATA_LOSS    # misaligned offset
    assert parse_code(with_tensor(0, [0], n_extra=64)) == L.DATA_LOSS              # empty dimension
    assert parse_code(with_tensor(0, [1, 1, 1, 1, 1], n_extra=64)) == L.DATA_LOSS  # five dimensions


def test_loader_refusals_without_a_device(tmp_path, model_dir):
    """load_native_llama's own checks come before any device work (src/pipeline/native_llama.cpp:10-55; tests/unit/test_metal_llama_decoder.cpp:610-614)."""
    from dooms_b200 import CudaLlamaDecoder

    def code_of(path, **kw):
        with pytest.raises(DoomsError) as e:
            CudaLlamaDecoder.load(str(path), **kw)
        return e.value.code
    assert code_of("/nonexistent/model.gguf") == L.NOT_FOUND
    assert code_of("/nonexistent/model.gguf", n_ctx=0) == L.INVALID_ARGUMENT
    junk = tmp_path / "junk.gguf"
    junk.write_bytes(b"not a gguf file at all")
    assert code_of(junk) == L.UNSUPPORTED
    good = write(model_dir, "loader_q4_0", synth.tiny_spec(QUANT_PLANS["q4_0"]), 11)
    assert code_of(good, n_ctx=4096) == L.INVALID_ARGUMENT          # beyond the model's context length (1024)

    def variant(name, **md_changes):
        spec = synth.tiny_spec(QUANT_PLANS["q4_0"])
        p = tmp_path / (name + ".gguf")
        synth.write_model(spec, p, 11)
        f = GgufFile(str(p))
        md = {"general.architecture": "qwen2", "qwen2.block_count": 2, "qwen2.embedding_length": 256, "qwen2.attention.head_count": 4,
              "qwen2.attention.head_count_kv": 2, "qwen2.feed_forward_length": 2304, "qwen2.context_length": 1024, "qwen2.rope.freq_base": 10000.0,
              "qwen2.attention.layer_norm_rms_epsilon": 1e-5}
        for k, v in md_changes.items():
            if v is None:
                md.pop(k, None)
            else:
                md[k] = v
        tensors = [(t["name"], t["dtype"], t["shape"], (lambda n=t["name"]: f.tensor_bytes(n))) for t in f.tensors()]
        GgufWriter().write(p.with_suffix(".v.gguf"), md, tensors)
        return p.with_suffix(".v.gguf")
    assert code_of(variant("arch", **{"general.architecture": "gpt2"})) == L.UNSUPPORTED
    assert code_of(variant("scaling", **{"qwen2.rope.scaling.type": "yarn"})) == L.UNSUPPORTED
    assert code_of(variant("nobase", **{"qwen2.rope.freq_base": None})) == L.INVALID_ARGUMENT
    assert code_of(variant("rotdim", **{"qwen2.rope.dimension_count": 32})) == L.UNSUPPORTED
    assert code_of(variant("heads", **{"qwen2.attention.head_count": 3})) == L.INVALID_ARGUMENT
