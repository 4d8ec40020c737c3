"""GGUF reader: CPU parse of a synthetic file (same results as the reference's reader, checked when
the reference checkout is present), and on the GPU a ternary tensor straight into a BitLinear layer."""
import os
import sys

import numpy as np
import pytest

from gguf_writer import synthetic_tensors, write_gguf
from oracle import bitlinear_np as O

REF_SRC = os.path.join(os.environ.get("ROTOR_RAG_REF", ""), "src")  # set ROTOR_RAG_REF to the reference checkout


def _check(reader, tensors):
    assert reader.version == 3 and reader.tensor_count == 4 and reader.metadata_count == 14
    md = reader.metadata
    assert md["general.architecture"] == "bitnet" and md["bitnet.block_count"] == 1 and md["flag"] is True
    assert md["general.file_type"] == -3 and md["u64"] == 1 << 40 and md["i64"] == -(1 << 40) and md["f64"] == 2.5
    assert abs(md["bitnet.rope.freq_base"] - 500000.0) < 1e-3 and md["tokenizer.ggml.tokens"] == ["<s>", "</s>", "hello"]
    assert reader.list_tensors() == list(tensors)
    for name, (tt, dims, data, _) in tensors.items():
        t = reader.get_tensor(name)
        assert list(t.dims) == dims and int(t.type) == tt
        assert np.array_equal(reader.load_tensor_data(name), data)
    with pytest.raises(ValueError):
        reader.load_tensor_data("missing")


def test_reader_parses_synthetic_file(tmp_path):
    from rotor_b200.gguf_parser import GGUFReader
    path = str(tmp_path / "tiny.gguf")
    tensors = write_gguf(path)
    _check(GGUFReader(path).read(), tensors)
    with open(tmp_path / "bad.gguf", "wb") as f:
        f.write(b"GGML" + b"\0" * 64)
    with pytest.raises(ValueError):
        GGUFReader(str(tmp_path / "bad.gguf")).read()


@pytest.mark.skipif(not os.path.isdir(REF_SRC), reason="reference checkout not present")
def test_reference_reader_agrees(tmp_path):
    """The unmodified reference reader sees the same file the same way."""
    import contextlib
    import io
    sys.path.insert(0, REF_SRC)
    try:
        from rotor.gguf_parser import GGUFReader as RefReader
    finally:
        sys.path.remove(REF_SRC)
    path = str(tmp_path / "tiny.gguf")
    tensors = write_gguf(path)
    ref = RefReader(path)
    with contextlib.redirect_stdout(io.StringIO()):
        ref.read()
    _check(ref, tensors)


@pytest.mark.gpu
def test_ternary_tensor_into_bitlinear(tmp_path):
    from rotor_b200.gguf_parser import GGUFReader
    from rotor_b200.transformer import TernaryLinear
    path = str(tmp_path / "tiny.gguf")
    tensors = write_gguf(path)
    reader = GGUFReader(path).read()
    name = "blk.0.attn_q.weight"
    w = tensors[name][3]
    lin = reader.load_linear(name, TernaryLinear(128, 48), scale=0.02)
    x = np.random.default_rng(2).standard_normal((3, 128)).astype(np.float32)
    want = O.bitlinear_float(x, w, 0.02)
    got = lin.forward(x)
    assert np.max(np.abs(got - want)) / np.sqrt(np.mean(want ** 2)) < 1e-3
    assert np.array_equal(lin.weights_cache, w)
    with pytest.raises(ValueError):
        reader.load_linear("token_embd.weight", TernaryLinear(16, 10))
