"""GGUF reader (jitllm_b200/gguf.py) on files written here: tensor table, alignment, key/values, refusals.
The refusals follow the reference reader's (convert/gguf/gguf.go:73-182)."""
import struct

import numpy as np
import pytest

from jitllm_b200 import synth
from jitllm_b200._lib import F32, MXFP4, Q4_K, Q8_0
from jitllm_b200.gguf import GGUFError, GGUFReader, write_gguf


def _model(tmp_path, alignment=32, version=3):
    rng = synth.rng_for(21)
    t = {
        "blk.0.attn_q.weight": (Q4_K, [512, 48], synth.q4k_matrix(rng, 48, 512).tobytes()),
        "blk.0.attn_k.weight": (Q8_0, [256, 24], synth.q8_0_matrix(rng, 24, 256).tobytes()),
        "blk.0.ffn_gate_exps.weight": (MXFP4, [64, 32, 4], synth.mxfp4_matrix(rng, 4 * 32, 64).tobytes()),
        "output_norm.weight": (F32, [512], np.ones(512, np.float32).tobytes()),
    }
    kv = {"general.architecture": "llama", "llama.block_count": 1, "llama.rope.freq_base": 500000.0,
          "tokenizer.ggml.tokens": ["a", "bc", ""], "general.flag": True, "llama.some_list": [1, 2, 3]}
    p = str(tmp_path / "m.gguf")
    write_gguf(p, kv, t, alignment=alignment, version=version)
    return p, t, kv


@pytest.mark.parametrize("alignment,version", [(32, 3), (64, 3), (256, 2)])
def test_round_trip(tmp_path, alignment, version):
    p, t, kv = _model(tmp_path, alignment, version)
    with GGUFReader(p) as r:
        assert r.version == version and r.alignment == alignment and r.data_start % alignment == 0
        assert r.kv["general.architecture"] == "llama" and r.kv["llama.block_count"] == 1
        assert r.kv["tokenizer.ggml.tokens"] == ["a", "bc", ""] and r.kv["llama.some_list"] == [1, 2, 3]
        assert r.kv["general.flag"] is True and abs(r.kv["llama.rope.freq_base"] - 500000.0) < 1e-3
        assert list(r.tensors) == list(t)                                   # file order kept
        for name, (typ, dims, data) in t.items():
            assert r.tensors[name]["type"] == typ and r.tensors[name]["dims"] == dims
            assert r.tensors[name]["offset"] % alignment == 0
            got = r.tensor_bytes(name)
            assert got.tobytes() == data
            del got
        assert r.matrix_shape("blk.0.attn_q.weight") == (1, 48, 512)
        assert r.matrix_shape("blk.0.ffn_gate_exps.weight") == (4, 32, 64)
        with pytest.raises(GGUFError):
            r.matrix_shape("output_norm.weight")


def test_decoded_tensor_matches_the_oracle(tmp_path, orc):
    p, t, _ = _model(tmp_path)
    with GGUFReader(p) as r:
        raw = r.tensor_bytes("blk.0.attn_q.weight")
        want = orc.dequant32(Q4_K, np.frombuffer(t["blk.0.attn_q.weight"][2], np.uint8), 48 * 512)
        assert np.array_equal(orc.dequant32(Q4_K, np.array(raw), 48 * 512), want)
        del raw


def test_refusals(tmp_path):
    p, _, _ = _model(tmp_path)
    blob = open(p, "rb").read()

    def reject(data, what):
        q = str(tmp_path / "bad.gguf")
        open(q, "wb").write(data)
        with pytest.raises(GGUFError, match=what):
            GGUFReader(q)
    reject(b"GGUX" + blob[4:], "not a GGUF")
    reject(blob[:4] + struct.pack("<I", 7) + blob[8:], "unsupported version")
    reject(blob[:8] + struct.pack("<Q", 10 ** 9) + blob[16:], "cannot fit")           # absurd tensor count
    reject(blob[:60], "truncated|runs past|cannot fit")
    reject(blob[:-100], "runs past the end")                                            # last tensor cut short
    # k that does not tile the block
    q = str(tmp_path / "odd.gguf")
    write_gguf(q, {}, {"w": (Q4_K, [512, 2], b"\0" * 576)})
    data = bytearray(open(q, "rb").read())
    i = data.index(b"w") + 1 + 4                     # name, n_dims -> first dim
    data[i:i + 8] = struct.pack("<Q", 500)
    open(q, "wb").write(bytes(data))
    with GGUFReader(q) as r:
        assert r.tensors["w"]["nbytes"] is None
        with pytest.raises(GGUFError):
            r.tensor_bytes("w")
    # duplicate names
    q2 = str(tmp_path / "dup.gguf")
    write_gguf(q2, {}, {"aa": (F32, [4], b"\0" * 16), "ab": (F32, [4], b"\0" * 16)})
    data = open(q2, "rb").read().replace(b"ab", b"aa")
    open(q2, "wb").write(data)
    with pytest.raises(GGUFError, match="duplicate"):
        GGUFReader(q2)
    # alignment that is not a power of two
    q3 = str(tmp_path / "al.gguf")
    write_gguf(q3, {"general.alignment": 48}, {"aa": (F32, [4], b"\0" * 16)})
    with pytest.raises(GGUFError, match="power of two"):
        GGUFReader(q3)
