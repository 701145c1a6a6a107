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


def _hf_files(tmp, kind):
    import synth
    spec = synth.spec_gpt2_tiny() if kind == "gpt2" else synth.spec_qwen_tiny()
    hf = synth.lm_tensors_hf(spec, 4321)
    names = list(hf)
    dtypes = {n: ("F32", "F16", "BF16")[i % 3] for i, n in enumerate(names)}
    paths = {}
    for tag, dt in (("f32", "F32"), ("mixed", dtypes)):
        p = os.path.join(tmp, f"{kind}_{tag}.safetensors")
        synth.write_safetensors(p, hf, dt, metadata={"format": "pt", "note": 'quotes " and \\ and {braces}'})
        paths[tag] = p
    return spec, paths


@pytest.mark.parametrize("kind", ["gpt2", "qwen"])
def test_safetensors_rules_match_the_reference_converters(tmp_path, kind):
    """oracle.safetensors_import_rules (which the GPU import is compared with) against the reference's own offline
    converters, tools/gpt2import.c and tools/qwenimport.c, built unchanged into oracle/_ref."""
    import subprocess
    tool = os.path.join(os.path.dirname(helpers.REF_LIB), f"{kind}import")
    if not os.path.exists(tool):
        pytest.skip("reference converters not built")
    from test_gpu_parity import _read_ncm
    spec, paths = _hf_files(str(tmp_path), kind)
    (tmp_path / "vocab.json").write_text("{}")
    (tmp_path / "tokenizer.json").write_text('{"model": {"vocab": {}, "merges": []}, "added_tokens": []}')
    (tmp_path / "merges.txt").write_text("#version: 0.2\n")
    for tag, p in paths.items():
        out = tmp_path / f"out_{tag}"
        out.mkdir()
        second = "vocab.json" if kind == "gpt2" else "tokenizer.json"
        subprocess.run([tool, p, str(tmp_path / second), str(tmp_path / "merges.txt"), str(out)],
                       capture_output=True, timeout=120)            # the tokenizer half may reject the empty vocabulary
        assert (out / "model.ncm").exists(), tag
        ref = _read_ncm(str(out / "model.ncm"))
        mine = orc.safetensors_import_rules(p, kind == "gpt2")
        assert list(ref) == list(mine), tag
        for n in ref:
            assert helpers.same_bits(ref[n], mine[n]), (tag, n)
    # and the f32 file converts back to the tensors the NCM1 writer emits for the same spec
    import synth
    direct = synth.lm_tensors(spec, 4321)
    mine = orc.safetensors_import_rules(paths["f32"], kind == "gpt2")
    assert set(mine) == set(direct)
    for n in direct:
        assert helpers.same_bits(mine[n], np.ascontiguousarray(direct[n], np.float32)), n
