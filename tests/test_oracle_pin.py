"""Pins the CPU oracle bit-for-bit.

1. Against committed golden vectors (tests/golden/golden.npz) produced by the
   reference's own CPU build on seeded inputs (tests/golden/make_golden.py).
2. Against that build itself when oracle/_ref/libcncm_ref.so is present (the
   container with the reference sources), on an extra case not in the file.
"""
import os

import numpy as np
import pytest

import helpers
import orc


@pytest.fixture(scope="module")
def golden():
    return dict(np.load(helpers.GOLDEN))


@pytest.fixture(scope="module")
def oracle_out(tmp_path_factory):
    out = {}
    tmp = str(tmp_path_factory.mktemp("orc"))
    helpers.orc_kernels(out)
    helpers.orc_ncp(out, tmp)
    helpers.orc_lms(out, tmp)
    return out


def test_oracle_library_builds():
    assert os.path.exists(orc.build())


def test_generated_weights_match_the_golden_run(golden, oracle_out):
    shas = [k for k in golden if k.startswith("sha_")]
    assert shas
    for k in shas:
        assert helpers.same_bits(golden[k], oracle_out[k]), (
            f"{k}: seeded weights differ from the run that produced the golden vectors")


def test_oracle_reproduces_every_golden_vector(golden, oracle_out):
    keys = [k for k in golden if not k.startswith("sha_")]
    assert len(keys) > 100
    missing = [k for k in keys if k not in oracle_out]
    assert not missing, missing
    bad = [k for k in keys if not helpers.same_bits(golden[k], oracle_out[k])]
    assert not bad, f"oracle differs from the reference on: {bad}"


@pytest.mark.skipif(not os.path.exists(helpers.REF_LIB), reason="reference build not present")
def test_oracle_matches_live_reference_on_a_fresh_case(tmp_path):
    import capi
    import cases
    import synth
    ref = capi.NcmLib(helpers.REF_LIB)
    spec = synth.spec_tiny(name="tiny_fresh", n_layer=3, n_embd=96, n_head=6, n_kv_heads=3,
                           prefix_len=17, mlp_hidden=80)
    conf, w = synth.write_ncp(spec, str(tmp_path), seed=99)
    pre, _, _ = cases.ncp_inputs(spec, B=5, seed=21)
    kw = cases.sampler_kwargs("cfg_pen", spec)
    got = orc.Model(conf, w).generate(pre, **kw)
    want = capi.NcpModel(ref, conf, w, arena_mb=256).generate(pre, **kw)
    assert (got == want).all()


def _ckpt_tensors():
    rng = np.random.default_rng(5)
    return {"wte.weight": rng.standard_normal((7, 5)).astype(np.float32),
            "h.0.ln_1.bias": rng.standard_normal(5).astype(np.float32),
            "conv.weight": rng.standard_normal((3, 4, 2)).astype(np.float32)}


@pytest.mark.skipif(not os.path.exists(helpers.REF_LIB), reason="reference build not present")
def test_checkpoint_writer_is_read_by_the_reference(tmp_path):
    """The NCK1 files the GPU tests feed to the library are files the reference's own reader accepts
    (weights_load -> ckpt_load_weights_only, src/tensor.c:73-80, src/ckpt.c:549-625) and reads the same tensors from."""
    import capi
    import synth
    ref = capi.NcmLib(helpers.REF_LIB)
    tensors = _ckpt_tensors()
    ck = str(tmp_path / "w.nckpt")
    synth.write_nck1(ck, tensors)
    assert ref.ckpt_probe(ck.encode()) == 1
    ws = ref.load_weights(ck)
    assert ws.count == len(tensors)
    for name, want in tensors.items():
        assert helpers.same_bits(ref.tensor_host(ws, name), want), name
    # a flipped payload byte is caught by the checksum
    raw = bytearray(open(ck, "rb").read())
    raw[len(raw) // 2] ^= 0x40
    bad = str(tmp_path / "bad.nckpt")
    open(bad, "wb").write(raw)
    with pytest.raises(RuntimeError):
        ref.load_weights(bad)
