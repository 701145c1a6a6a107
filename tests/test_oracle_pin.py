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
