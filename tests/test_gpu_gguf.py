"""Tensors read out of a GGUF file and uploaded as they are: decode parity against the oracle on the same bytes."""
import numpy as np
import pytest

from conftest import parity_err
from jitllm_b200 import synth
from jitllm_b200._lib import MXFP4, Q4_K, Q8_0
from jitllm_b200.gguf import GGUFReader, write_gguf

pytestmark = pytest.mark.gpu


def test_upload_from_gguf_and_decode(dev, orc, tmp_path):
    import torch
    rng = synth.rng_for(31)
    mats = {"q.weight": (Q4_K, 96, 1024, synth.q4k_matrix(rng, 96, 1024)),
            "k.weight": (Q8_0, 64, 512, synth.q8_0_matrix(rng, 64, 512)),
            "exps.weight": (MXFP4, 3 * 32, 128, synth.mxfp4_matrix(rng, 3 * 32, 128))}
    p = str(tmp_path / "m.gguf")
    write_gguf(p, {"general.architecture": "test"},
               {"q.weight": (Q4_K, [1024, 96], mats["q.weight"][3].tobytes()),
                "k.weight": (Q8_0, [512, 64], mats["k.weight"][3].tobytes()),
                "exps.weight": (MXFP4, [128, 32, 3], mats["exps.weight"][3].tobytes())})
    with GGUFReader(p) as r:
        for name in ("q.weight", "k.weight"):
            t, rows, k, w = mats[name]
            h = r.upload(dev, name)
            assert (h.nrows, h.k) == (rows, k)
            x = synth.activations(rng, 1, k)
            out = torch.empty(1, rows, device="cuda")
            dev.Reserve(rows, k, 1)
            dev.MatVecDev(out, h, torch.from_numpy(x).cuda(), 1, torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert parity_err(out.cpu().numpy(), orc.matmul_f64(t, w, x, rows, k, 1)) <= 2e-3
            h.free()
        bank = r.upload(dev, "exps.weight")
        assert (bank.n_expert, bank.nrows, bank.k) == (3, 32, 128)
        bank.free()
