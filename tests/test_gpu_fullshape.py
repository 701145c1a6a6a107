"""Parity at the stated shapes of the five configurations, through the C ABI, against the CPU oracle.

The other GPU tests use models the oracle finishes in a fraction of a second; error grows with depth and
with the length of the contractions, so these run the real widths and depths on a handful of rows:

* config 2 at its 12 layers, sampled as configured (CFG 1.5, temp 0.8, top-k 50, top-p 0.9, frequency 0.2);
* config 1b (ladder 1-3-9-81) at 64 sequences, greedy, codes and the 81 decoded tokens;
* config 5's widths (d = 1024, 16 query / 4 kv heads, 16 384 codes) at 2 layers;
* the GPT-2 124M shape: logits of a 128-id prompt, greedy ids alone and inside a batch of 64;
* the Qwen2-0.5B shape with bf16-rounded weights: logits of a 64-id prompt, greedy ids, and sampled ids
  at temp 0.7 / top-p 0.95 over the 151 936-entry vocabulary.

Bars: integer results equal the oracle's; a differing greedy id is accepted only when the oracle's two
largest logits at that step lie within 1e-5 relative (counted and printed); logits within 1e-3 max-abs.
The oracle needs a few minutes of host time for this file.
"""
import os

import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu

ATOL_LOGITS = 1e-3
NEAR_TIE = 1e-5
# sampled ids: the nucleus walk goes down the sorted probabilities until the running sum passes the draw, so which
# of two neighbours of that order it stops at moves with the logits' last bits; over 151 936 near-uniform
# probabilities neighbours are ~1e-5 apart in logit. A differing id is accepted only if the oracle's logits of the
# two ids are closer than this (a tenth of the logits tolerance), and is counted.
NEAR_TIE_SAMPLED = 1e-4


@pytest.fixture(scope="module")
def cuda():
    import capi
    if not os.path.exists(helpers.CUDA_LIB):
        pytest.fail("libncm_b200.so is not built: run python saphira-cncm_b200/build.py")
    lib = capi.NcmLib(helpers.CUDA_LIB)
    lib.ncmb_set_gemm_mode(int(os.environ.get("NCM_TEST_GEMM", "3")))
    return lib


@pytest.fixture(scope="module")
def tmp(tmp_path_factory):
    return str(tmp_path_factory.mktemp("full"))


def _max_err(name, got, want, atol, rtol=1e-5):
    assert got.shape == want.shape, name
    fin = np.isfinite(want)
    assert (np.isfinite(got) == fin).all(), f"{name}: non-finite pattern differs"
    d = np.abs(got[fin].astype(np.float64) - want[fin])
    over = d - (atol + rtol * np.abs(want[fin]))
    assert over.max() <= 0, f"{name}: max abs err {d.max():.3e} exceeds {atol:.1e} + {rtol:.0e}*|x|"
    return float(d.max())


_top2_gap = helpers.top2_gap


def _level_offsets(spec, with_l0=True):
    """(offset, vocabulary) of every sampled position inside a captured logits row"""
    offs, o = [], 0
    for k in range(0 if with_l0 else 1, len(spec.levels)):
        for _ in range(spec.levels[k]):
            offs.append((o, spec.vocab[k]))
            o += spec.vocab[k]
    return offs, o


def _gen_kwargs(spec):
    g = dict(spec.gen)
    kw = dict(temp=g.get("temperature", 0.0), top_k=g.get("top_k", 0), top_p=g.get("top_p", 1.0),
              cfg=g.get("cfg_scale", 0.0), freq=g.get("freq", 0.0), mu=g.get("mu", 0.0))
    if spec.token_unigram:
        kw["allow"] = np.full(max(spec.vocab), 1.0 / max(spec.vocab))
    return kw


def _sampled_rows(got, want, lg_g, lg_o, spec, tag):
    """Sampled codes: rows must be identical. A differing row is accepted (and counted) only when, at its first
    differing position, both libraries' logits agree within the logit bound and the two picks are neighbours in
    the oracle's sorted order (the nucleus walk stopped one entry apart) or sit at the top-k boundary."""
    offs, _ = _level_offsets(spec)
    near = []
    for b in np.nonzero((got != want).any(axis=1))[0]:
        j = int(np.nonzero(got[b] != want[b])[0][0])
        off, V = offs[j]
        ro, rg = lg_o[b, off:off + V], lg_g[b, off:off + V]
        assert np.abs(ro - rg).max() <= ATOL_LOGITS, f"{tag}: row {b} differs at code {j} with logits apart"
        order = np.argsort(-ro, kind="stable")
        rank = {int(v): i for i, v in enumerate(order[:256])}
        ra, rb = rank.get(int(got[b, j]), 10 ** 6), rank.get(int(want[b, j]), 10 ** 6)
        assert abs(ra - rb) == 1, f"{tag}: row {b} code {j}: picks {got[b, j]} / {want[b, j]} are not neighbours (ranks {ra}, {rb})"
        near.append(int(b))
    print(f"{tag}: {got.shape[0] - len(near)}/{got.shape[0]} rows identical, {len(near)} differ at a walk boundary")
    return near


def test_c2_at_full_depth_sampled_as_configured(cuda, tmp):
    import capi
    import orc
    import synth
    spec = synth.spec_c2()
    assert spec.n_layer == 12 and spec.n_embd == 512
    conf, w = synth.write_ncp(spec, tmp)
    B = 4
    pre = synth.ncp_prefixes(spec, B, 11)
    pre[1, -40:] = spec.pad_id                           # one row with trailing pads
    kw = _gen_kwargs(spec)
    assert kw["cfg"] == 1.5 and kw["top_k"] == 50
    om = orc.Model(conf, w)
    _, cap = _level_offsets(spec)
    want, lg_o = om.generate(pre, seed=5, cap_floats=cap, **kw)
    gm = capi.NcpModel(cuda, conf, w, arena_mb=64)
    got, lg_g = gm.generate_ex(pre, cap, seed=5, **kw)
    assert cuda.ncmb_gemm_tc_check() == 0
    n0 = spec.levels[0] * spec.vocab[0]
    e0 = _max_err("c2 level-0 logits", lg_g[:, :n0], lg_o[:, :n0], ATOL_LOGITS)
    near = _sampled_rows(got, want, lg_g, lg_o, spec, "c2 x12")
    assert len(near) <= 1
    same = (got == want).all(axis=1)
    e = _max_err("c2 logits", lg_g[same], lg_o[same], ATOL_LOGITS)
    print(f"c2 x12: logits max abs err level 0 {e0:.2e}, all levels {e:.2e}")
    helpers.decoded_tokens_equal_or_near_tie(gm, om, want, spec, "c2 x12")


def test_c1b_ladder_1_3_9_81_greedy_codes_and_81_tokens(cuda, tmp):
    import capi
    import orc
    import synth
    from test_gpu_parity import _near_tie_rows
    spec = synth.spec_c1((1, 3, 9, 81))
    conf, w = synth.write_ncp(spec, tmp)
    B = 64
    pre = synth.ncp_prefixes(spec, B, 7)
    om = orc.Model(conf, w)
    _, cap = _level_offsets(spec)
    want, lg_o = om.generate(pre, temp=0.0, cap_floats=cap)
    gm = capi.NcpModel(cuda, conf, w, arena_mb=64)
    got, lg_g = gm.generate_ex(pre, cap, temp=0.0)
    ex, un = _near_tie_rows(got, want, lg_o, spec, with_l0=True)
    print(f"c1b greedy B={B}: {len(ex)} near-tie rows, {len(un)} unexplained")
    assert not un, f"rows differ without a near-tie: {un}"
    same = (got == want).all(axis=1)
    _max_err("c1b logits", lg_g[same], lg_o[same], ATOL_LOGITS)
    tok = helpers.decoded_tokens_equal_or_near_tie(gm, om, want, spec, "c1b")
    assert tok.shape == (B, 81)


def test_c5_widths_at_two_layers(cuda, tmp):
    import capi
    import orc
    import synth
    spec = synth.spec_c2(n_layer=2, n_embd=1024, n_head=16, n_kv=4, vocab=16384, name="c5_l2")
    conf, w = synth.write_ncp(spec, tmp)
    B = 2
    pre = synth.ncp_prefixes(spec, B, 13)
    pre[0, -17:] = spec.pad_id
    kw = _gen_kwargs(spec)
    om = orc.Model(conf, w)
    _, cap = _level_offsets(spec)
    want, lg_o = om.generate(pre, seed=3, cap_floats=cap, **kw)
    gm = capi.NcpModel(cuda, conf, w, arena_mb=64)
    got, lg_g = gm.generate_ex(pre, cap, seed=3, **kw)
    assert cuda.ncmb_gemm_tc_check() == 0
    near = _sampled_rows(got, want, lg_g, lg_o, spec, "c5 widths")
    assert not near
    e = _max_err("c5 logits", lg_g, lg_o, ATOL_LOGITS)
    print(f"c5 widths x2 layers: logits max abs err {e:.2e}")
    helpers.decoded_tokens_equal_or_near_tie(gm, om, want, spec, "c5 widths")


def _greedy_ids_or_near_tie(om, prompt, got, tag):
    """got: ids the library generated greedily after `prompt`. Walks the oracle step by step on the library's own
    ids; a step where they part is accepted only as a near-tie of the oracle's two largest logits."""
    ids = list(map(int, prompt))
    ties = 0
    for i, g in enumerate(got):
        lg = om.logits(np.array(ids, np.int32), last_only=True)
        w = int(np.argmax(lg))
        if g != w:
            gap = _top2_gap(lg)
            assert gap <= NEAR_TIE and g in np.argsort(lg)[-2:], f"{tag}: id {i} is {g}, oracle {w}, top-2 gap {gap:.2e}"
            ties += 1
        ids.append(int(g))
    return ties


def _sampled_ids_or_near_tie(om, prompt, got, temp, top_k, top_p, seed, tag):
    """got: ids the library sampled after `prompt` with the reference's generator (one draw per id). Walks the oracle
    step by step on the library's own ids and the same draws; a step where they part is accepted only between two
    ids whose oracle logits are within NEAR_TIE_SAMPLED."""
    import orc
    ids = list(map(int, prompt))
    state, ties = seed, 0
    for i, g in enumerate(got):
        lg = om.logits(np.array(ids, np.int32), last_only=True)
        w, state = orc.sample_topkp(lg.copy(), temp, top_k, top_p, state)
        if g != w:
            gap = abs(float(lg[g]) - float(lg[w]))
            assert gap <= NEAR_TIE_SAMPLED, f"{tag}: id {i} is {g}, oracle {w}, their logits {gap:.2e} apart"
            ties += 1
        ids.append(int(g))
    return ties


def test_gpt2_124m_shape_logits_and_greedy_ids(cuda, tmp):
    import orc
    import synth
    spec = synth.spec_gpt2_124m()
    assert (spec.n_layer, spec.n_embd, spec.vocab) == (12, 768, 50257)
    conf, w = synth.write_lm(spec, tmp)
    cfg = cuda.load_config(conf)
    m = cuda.ncmb_lm_open(cfg, w.encode(), 0, 0)
    assert m
    om = orc.LM(conf, w, False)
    B, P, n_new = 64, 128, 8
    prompts = np.ascontiguousarray(synth.lm_prompts(spec, B, P, 3))
    pr = prompts[0]
    lg = np.zeros((P, spec.vocab), np.float32)
    cuda.ncmb_lm_logits(m, pr.ctypes.data, P, 0, lg.ctypes.data)
    e = _max_err("gpt2-124m logits", lg, om.logits(pr), ATOL_LOGITS)
    print(f"gpt2 124M shape: logits of a {P}-id prompt, max abs err {e:.2e}")
    # one sequence (weight-streaming decode steps)
    out1 = np.zeros((1, n_new), np.int32)
    cuda.ncmb_lm_generate(m, pr.ctypes.data, 1, P, n_new, 0.0, 0, 1.0, 0, -1, out1.ctypes.data)
    ties = _greedy_ids_or_near_tie(om, pr, out1[0], "gpt2 B=1")
    # 64 sequences (tensor-core decode steps); three of the rows are checked
    out = np.zeros((B, n_new), np.int32)
    cuda.ncmb_lm_generate(m, prompts.ctypes.data, B, P, n_new, 0.0, 0, 1.0, 0, -1, out.ctypes.data)
    assert cuda.ncmb_gemm_tc_check() == 0
    for b in (0, 17, 63):
        ties += _greedy_ids_or_near_tie(om, prompts[b], out[b], f"gpt2 B=64 row {b}")
    print(f"gpt2 124M shape: {n_new} greedy ids at B=1 and 3 rows of B=64, {ties} near-ties")
    cuda.ncmb_lm_close(m)


def test_qwen2_05b_shape_bf16_weights_logits_greedy_and_sampled_ids(cuda, tmp):
    import orc
    import synth
    spec = synth.spec_qwen_05b()
    assert (spec.n_layer, spec.n_embd, spec.vocab, spec.bf16_round) == (24, 896, 151936, 1)
    conf, w = synth.write_lm(spec, tmp)
    cfg = cuda.load_config(conf)
    m = cuda.ncmb_lm_open(cfg, w.encode(), 1, 1)
    assert m
    om = orc.LM(conf, w, True)
    P, n_new = 64, 8
    pr = np.ascontiguousarray(synth.lm_prompts(spec, 1, P, 3)[0])
    lg = np.zeros((P, spec.vocab), np.float32)
    cuda.ncmb_lm_logits(m, pr.ctypes.data, P, 0, lg.ctypes.data)
    e = _max_err("qwen2-0.5b logits", lg, om.logits(pr), ATOL_LOGITS)
    print(f"qwen2 0.5B shape: logits of a {P}-id prompt, max abs err {e:.2e}")
    out = np.zeros((1, n_new), np.int32)
    cuda.ncmb_lm_generate(m, pr.ctypes.data, 1, P, n_new, 0.0, 0, 1.0, 0, -1, out.ctypes.data)
    ties = _greedy_ids_or_near_tie(om, pr, out[0], "qwen B=1")
    print(f"qwen2 0.5B shape: {n_new} greedy ids, {ties} near-ties")
    # the configuration's sampler over the whole vocabulary (device-wide sort of 151 936 entries): two ids
    n_s = 2
    outs = np.zeros((1, n_s), np.int32)
    cuda.ncmb_lm_generate(m, pr.ctypes.data, 1, P, n_s, 0.7, 0, 0.95, 9, -1, outs.ctypes.data)
    assert cuda.ncmb_gemm_tc_check() == 0
    ties = _sampled_ids_or_near_tie(om, pr, outs[0], 0.7, 0, 0.95, 9, "qwen sampled")
    print(f"qwen2 0.5B shape: {n_s} sampled ids, {ties} near-ties")
    cuda.ncmb_lm_close(m)
    try:
        os.remove(w)                                       # 2 GB of weights
    except OSError:
        pass
