"""Parity of the CUDA library with the CPU oracle, through the C ABI.

Integer results (codes, picks, token ids, nearest-code indices) must be equal;
a differing row is accepted only when the logits it was drawn from show a
near-tie (top-2 gap within 1e-5 relative), and such rows are counted and
printed.  Floating-point stages are compared with the tolerance written beside
each check (the headline bound is 1e-3 max-abs on logits in fp32 mode).
"""
import os

import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu

ATOL_KERNEL = 2e-5       # single layer kernels, inputs in [-2, 2]
ATOL_STAGE = 1e-4        # quantizer / VQ-VAE stage tensors
ATOL_LOGITS = 1e-3       # logits, fp32 mode


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
    return str(tmp_path_factory.mktemp("gpu"))


def _cmp_float(name, got, want, atol, rtol=1e-5):
    """|got - want| <= atol + rtol * |want| element-wise; returns the max abs error."""
    assert got.shape == want.shape, name
    fin = np.isfinite(want)
    assert (np.isfinite(got) == fin).all(), f"{name}: non-finite pattern differs"
    if not fin.any():
        return 0.0
    d = np.abs(got[fin].astype(np.float64) - want[fin])
    over = d - (atol + rtol * np.abs(want[fin]))
    assert over.max() <= 0, f"{name}: max abs err {d.max():.3e} exceeds {atol:.1e} + {rtol:.0e}*|x|"
    return float(d.max())


def test_layer_kernels_match_oracle(cuda):
    got, want = {}, {}
    helpers.capi_kernels(cuda, got)
    helpers.orc_kernels(want)
    for k in want:
        if want[k].dtype.kind in "iu":
            assert (got[k] == want[k]).all(), k
        else:
            _cmp_float(k, got[k], want[k], ATOL_KERNEL)


@pytest.mark.parametrize("variant", ["plain", "full", "tied", "shared", "norope_relu2", "given_l0", "causal"])
def test_ncp_variant_matches_oracle(cuda, tmp, variant):
    got, want = {}, {}
    helpers.capi_ncp(cuda, got, tmp, variants=[variant], with_c1=False)
    helpers.orc_ncp(want, tmp, variants=[variant], with_c1=False)
    bad = []
    for k in sorted(want):
        if k.startswith("sha_"):
            continue
        if want[k].dtype.kind in "iu":
            if not (got[k] == want[k]).all():
                bad.append((k, int((got[k] != want[k]).sum())))
        else:
            tol = ATOL_LOGITS if "logits" in k else ATOL_STAGE
            _cmp_float(k, got[k], want[k], tol)
    assert not bad, f"integer outputs differ from the oracle: {bad}"


@pytest.mark.parametrize("variant", ["full", "shared", "plain"])
def test_two_phase_sampler_picks_what_the_one_kernel_sampler_picks(cuda, tmp, variant):
    """Candidate selection for all positions at once + a sequential kernel over the candidates (used when penalties
    can only lower logits) against the oracle and against the one-kernel sampler, forced on at the tiny vocabularies."""
    import capi
    import cases
    import orc
    import synth
    spec = cases.ncp_spec(variant)
    conf, w = synth.write_ncp(spec, tmp)
    pre, l0, _ = cases.ncp_inputs(spec)
    om = orc.Model(conf, w)
    gm = capi.NcpModel(cuda, conf, w, arena_mb=64)
    try:
        for sname in ("topk", "cfg", "cfg_pen_down"):
            kw = cases.sampler_kwargs(sname, spec)
            if kw.get("cfg", 0) > 0 and spec.pad_id < 0:
                continue
            use_l0 = l0 if not spec.query_level0 else None
            want = om.generate(pre, l0=use_l0, **kw)
            for mode in ("1", "2"):
                os.environ["NCM_B200_SAMPLE_PHASES"] = mode
                got = gm.generate(pre, l0=use_l0, **kw)
                assert np.array_equal(got, want), (variant, sname, mode)
    finally:
        os.environ.pop("NCM_B200_SAMPLE_PHASES", None)


def _gen_kwargs(spec):
    g = dict(spec.gen)
    kw = dict(temp=g.get("temperature", 0.0), top_k=g.get("top_k", 0), top_p=g.get("top_p", 1.0),
              cfg=g.get("cfg_scale", 0.0), freq=g.get("freq", 0.0), mu=g.get("mu", 0.0))
    if spec.token_unigram:
        kw["allow"] = np.full(max(spec.vocab), 1.0 / max(spec.vocab))
    return kw


def _near_tie_rows(codes_g, codes_o, logits_o, spec, with_l0):
    """Rows that differ, split into explained-by-near-tie and unexplained.

    A differing row is explained when, at its first differing code, the oracle
    logits' top-2 gap is within 1e-5 relative (greedy) -- everything after that
    position legitimately diverges."""
    lv_first = 0 if with_l0 else 1
    offs, o = [], 0
    for k in range(lv_first, len(spec.levels)):
        V = spec.vocab[k]
        for t in range(spec.levels[k]):
            offs.append((o, V))
            o += V
    explained, unexplained = [], []
    code_base = 0 if with_l0 else spec.levels[0]
    for b in np.nonzero((codes_g != codes_o).any(axis=1))[0]:
        j = int(np.nonzero(codes_g[b] != codes_o[b])[0][0])
        if j < code_base:
            unexplained.append(int(b))
            continue
        off, V = offs[j - code_base]
        row = np.sort(logits_o[b, off:off + V])[::-1]
        gap = abs(row[0] - row[1]) / max(abs(row[0]), 1e-30)
        (explained if gap <= 1e-5 else unexplained).append(int(b))
    return explained, unexplained


def test_c1_full_batch_greedy_codes_and_tokens(cuda, tmp):
    import capi
    import orc
    import synth
    spec = synth.spec_c1()
    conf, w = synth.write_ncp(spec, tmp)
    B = 64
    pre = synth.ncp_prefixes(spec, B, 7)
    om = orc.Model(conf, w)
    cap = sum(l * v for l, v in zip(spec.levels, spec.vocab))
    want, lg_o = om.generate(pre, temp=0.0, cap_floats=cap)
    gm = capi.NcpModel(cuda, conf, w, arena_mb=64)
    got, lg_g = gm.generate_ex(pre, cap, temp=0.0)
    ex, un = _near_tie_rows(got, want, lg_o, spec, with_l0=True)
    print(f"c1 greedy B={B}: {len(ex)} near-tie rows, {len(un)} unexplained")
    assert not un, f"rows differ without a near-tie: {un}"
    same = (got == want).all(axis=1)
    _cmp_float("c1 logits", lg_g[same], lg_o[same], ATOL_LOGITS)
    helpers.decoded_tokens_equal_or_near_tie(gm, om, got, spec, "c1")


def test_c2_shape_reduced_depth_sampled_codes(cuda, tmp):
    """Config-2 widths (d=512, 8q/2kv heads, SwiGLU, CFG, top-k/top-p, cascade) at 2 layers, 3 rows."""
    import capi
    import orc
    import synth
    spec = synth.spec_c2(n_layer=2, name="c2_l2")
    conf, w = synth.write_ncp(spec, tmp)
    B = 3
    pre = synth.ncp_prefixes(spec, B, 11)
    pre[1, -40:] = spec.pad_id
    kw = _gen_kwargs(spec)
    om = orc.Model(conf, w)
    cap = sum(l * v for l, v in zip(spec.levels, spec.vocab))
    want, lg_o = om.generate(pre, seed=5, cap_floats=cap, **kw)
    gm = capi.NcpModel(cuda, conf, w, arena_mb=64)
    got, lg_g = gm.generate_ex(pre, cap, seed=5, **kw)
    same = (got == want).all(axis=1)
    print(f"c2-shaped: {int(same.sum())}/{B} rows identical")
    # level-0 logits do not depend on earlier picks: always comparable
    n0 = spec.levels[0] * spec.vocab[0]
    _cmp_float("c2 level-0 logits", lg_g[:, :n0], lg_o[:, :n0], ATOL_LOGITS)
    assert same.all(), (got, want)
    _cmp_float("c2 logits", lg_g, lg_o, ATOL_LOGITS)


def test_qkv_projection_with_norm_and_rotation_in_its_epilogue(cuda, tmp):
    """Opt-in path: the per-head RMSNorm and the rotary embedding applied by the QKV GEMM's epilogue (head dim 64)
    instead of a pass of their own. Same codes as the oracle, logits within the usual bound."""
    import capi
    import orc
    import synth
    spec = synth.spec_c2(n_layer=2, name="c2_l2_qkepi")
    conf, w = synth.write_ncp(spec, tmp)
    pre = synth.ncp_prefixes(spec, 3, 11)
    kw = _gen_kwargs(spec)
    cap = sum(l * v for l, v in zip(spec.levels, spec.vocab))
    want, lg_o = orc.Model(conf, w).generate(pre, seed=5, cap_floats=cap, **kw)
    gm = capi.NcpModel(cuda, conf, w, arena_mb=64)
    gm.generate_ex(pre, cap, seed=5, **kw)           # the first call also prepares the weights' fp16 pairs
    os.environ["NCM_B200_QK_EPILOGUE"] = "1"
    try:
        n0 = cuda.ncmb_launch_count()
        got, lg_g = gm.generate_ex(pre, cap, seed=5, **kw)
        fused = cuda.ncmb_launch_count() - n0
    finally:
        os.environ.pop("NCM_B200_QK_EPILOGUE", None)
    n0 = cuda.ncmb_launch_count()
    got2, _ = gm.generate_ex(pre, cap, seed=5, **kw)
    plain = cuda.ncmb_launch_count() - n0
    assert fused < plain                       # the separate norm / rotation launches are gone
    assert np.array_equal(got, want) and np.array_equal(got2, want)
    _cmp_float("logits, fused QKV epilogue", lg_g, lg_o, ATOL_LOGITS)


def test_stepper_equals_monolithic_and_is_deterministic(cuda, tmp):
    import ctypes as C
    import capi
    import cases
    spec = cases.ncp_spec("full")
    import synth
    conf, w = synth.write_ncp(spec, tmp)
    m = capi.NcpModel(cuda, conf, w, arena_mb=64)
    pre, _, _ = cases.ncp_inputs(spec)
    kw = cases.sampler_kwargs("cfg_pen", spec)
    a = m.generate(pre, **kw)
    b = m.generate(pre, **kw)
    assert (a == b).all()
    allow = np.ascontiguousarray(kw["allow"], dtype=np.float64)
    adj = kw["adj"]
    g = cuda.ncp_gen_begin(m.ncp, None, pre.ctypes.data, pre.shape[0], kw["temp"], kw["top_k"], kw["top_p"],
                           kw["cfg"], kw["freq"], kw["mu"], adj[0], adj[1], adj[2], allow.ctypes.data, kw["seed"])
    ns = cuda.ncp_gen_nsteps(g)
    assert ns == len(spec.levels)
    row0 = []
    buf = (C.c_int * 64)()
    n = C.c_int(0)
    for s in range(ns):
        assert cuda.ncp_gen_step(g, buf, C.byref(n)) == 0
        assert n.value == cuda.ncp_gen_step_size(g, s) == spec.levels[s]
        row0 += list(buf[:n.value])
    assert cuda.ncp_gen_step(g, None, None) == 1
    out = cuda.ncp_gen_finish(g)
    codes = np.ctypeslib.as_array(C.cast(out, C.POINTER(C.c_int)), shape=a.shape).copy()
    capi._libc.free(out)
    assert (codes == a).all()
    assert row0 == list(a[0])


def test_rows_do_not_depend_on_batch_composition(cuda, tmp):
    """Greedy codes of a row are the same alone, in a batch, and in a permuted batch."""
    import capi
    import synth
    spec = synth.spec_c1()
    conf, w = synth.write_ncp(spec, tmp)
    m = capi.NcpModel(cuda, conf, w, arena_mb=64)
    pre = synth.ncp_prefixes(spec, 16, 3)
    full = m.generate(pre, temp=0.0)
    perm = np.random.default_rng(0).permutation(16)
    assert (m.generate(pre[perm], temp=0.0) == full[perm]).all()
    assert (m.generate(pre[5:6], temp=0.0) == full[5:6]).all()


def test_quantizer_nearest_code_sweep(cuda, tmp):
    """Flat nearest-code search on N(0,1) vectors against a 4096 x 64 codebook."""
    import capi
    import orc
    import synth
    spec = synth.spec_c2(n_layer=1, name="c2_q")
    conf, w = synth.write_ncp(spec, tmp)
    m = capi.NcpModel(cuda, conf, w, arena_mb=64)
    rng = np.random.default_rng(5)
    n = 4096
    x = (rng.standard_normal((n, 64)) * 0.02).astype(np.float32)
    xd = cuda.to_backend(x)
    idx_d = cuda.alloc(n)
    cuda.ncmb_vq_nearest_dev(m.vq, 3, xd, n, idx_d)
    got = cuda.to_host(idx_d, (n,), np.int32)
    E = synth.ncp_tensors(spec, 1234)["tok.vq.embeddings.3.weight"]
    d = orc.l2sq(x, E)
    want = d.argmin(axis=1).astype(np.int32)
    diff = np.nonzero(got != want)[0]
    for i in diff:      # accept only near-ties of the two distances
        a, b = d[i, got[i]], d[i, want[i]]
        assert abs(a - b) <= 1e-5 * max(abs(b), 1e-30), (i, a, b)
    print(f"nearest-code: {len(diff)} near-ties of {n}")


def test_quantizer_sweep_box_scale_codebook(cuda, tmp):
    """N(0,1) vectors against a 16384 x 64 codebook (the box-scale sweep's shapes) on the tensor-core
    route; 512 sampled rows are checked against the oracle's distances."""
    import capi
    import orc
    import synth
    spec = synth.spec_c2(n_layer=1, vocab=16384, name="c5_q")
    conf, w = synth.write_ncp(spec, tmp)
    m = capi.NcpModel(cuda, conf, w, arena_mb=64)
    rng = np.random.default_rng(8)
    n = 1 << 16
    x = rng.standard_normal((n, 64)).astype(np.float32)
    xd, idx_d = cuda.to_backend(x), cuda.alloc(n)
    cuda.ncmb_vq_nearest_dev(m.vq, 2, xd, n, idx_d)
    got = cuda.to_host(idx_d, (n,), np.int32)
    assert cuda.ncmb_gemm_tc_check() == 0
    assert got.min() >= 0 and got.max() < 16384
    E = synth.ncp_tensors(spec, 1234)["tok.vq.embeddings.2.weight"]
    pick = rng.choice(n, 512, replace=False)
    d = orc.l2sq(x[pick], E)
    want = d.argmin(axis=1)
    ties = 0
    for r, i in enumerate(pick):
        if got[i] != want[r]:
            a, b = d[r, got[i]], d[r, want[r]]
            assert abs(a - b) <= 1e-5 * abs(b), (i, a, b)
            ties += 1
    print(f"box-scale nearest-code: {ties} near-ties in 512 sampled rows")


def test_generate_in_waves_equals_one_pass(cuda, tmp):
    """A batch that does not fit the GPU runs as waves of rows; sampled codes must not change (reference RNG stream
    sliced per wave, CFG rows kept with their sequences)."""
    import synth
    spec = synth.spec_tiny()
    conf, w = synth.write_ncp(spec, tmp)
    pre = synth.ncp_prefixes(spec, 7, 21)
    kw = dict(temp=0.9, top_k=6, top_p=0.95, cfg=1.3, freq=0.2, seed=77)
    import capi
    model = capi.NcpModel(cuda, conf, w)
    try:
        os.environ.pop("NCM_B200_WAVE_ROWS", None)
        one = model.generate(pre, **kw)
        for rows in (1, 3):
            os.environ["NCM_B200_WAVE_ROWS"] = str(rows)
            assert np.array_equal(model.generate(pre, **kw), one), rows
    finally:
        os.environ.pop("NCM_B200_WAVE_ROWS", None)


def test_counter_based_stream_makes_rows_independent_of_sharding(cuda, tmp):
    """With ncmb_set_rng_mode(1) a sequence's draws are keyed by (seed, global row, level, position): eight rows in
    one call, two calls of four with row offsets 0 / 4, eight single-row calls in reverse order and a run in waves
    of three all give the same codes, with CFG (whose unconditional twins sample level 0 too) and penalties on.
    The reference's batch-ordered stream (mode 0, the default) still equals the oracle afterwards."""
    import capi
    import cases
    import orc
    import synth
    spec = cases.ncp_spec("full")
    conf, w = synth.write_ncp(spec, tmp)
    m = capi.NcpModel(cuda, conf, w, arena_mb=64)
    pre = synth.ncp_prefixes(spec, 8, 31)
    pre[2, -4:] = spec.pad_id
    try:
        for sname in ("cfg_pen", "cfg_pen_down", "topk"):
            kw = cases.sampler_kwargs(sname, spec)
            cuda.ncmb_set_rng_mode(1)
            cuda.ncmb_set_row_offset(0)
            whole = m.generate(pre, **kw)
            assert not (whole[0] == whole[1:]).all()           # rows do differ from one another
            halves = []
            for off in (0, 4):
                cuda.ncmb_set_row_offset(off)
                halves.append(m.generate(pre[off:off + 4], **kw))
            assert np.array_equal(np.concatenate(halves), whole), sname
            for i in reversed(range(8)):
                cuda.ncmb_set_row_offset(i)
                assert np.array_equal(m.generate(pre[i:i + 1], **kw)[0], whole[i]), (sname, i)
            cuda.ncmb_set_row_offset(0)
            os.environ["NCM_B200_WAVE_ROWS"] = "3"
            assert np.array_equal(m.generate(pre, **kw), whole), sname
            os.environ.pop("NCM_B200_WAVE_ROWS", None)
            # another offset is another set of sequences
            cuda.ncmb_set_row_offset(100)
            assert not np.array_equal(m.generate(pre, **kw), whole)
            cuda.ncmb_set_row_offset(0)
            cuda.ncmb_set_rng_mode(0)
            assert np.array_equal(m.generate(pre, **kw), orc.Model(conf, w).generate(pre, **kw)), sname
    finally:
        os.environ.pop("NCM_B200_WAVE_ROWS", None)
        cuda.ncmb_set_rng_mode(0)
        cuda.ncmb_set_row_offset(0)


LM_SPECS = {
    # head dim 16: every kernel of the generic path (GEMV, split-key attention, CUDA graph replay)
    "gpt2": lambda synth: synth.spec_gpt2_tiny(),
    "qwen": lambda synth: synth.spec_qwen_tiny(),
    # head dim 64 (the decode-attention and GEMV kernels at the models' real head size)
    "gpt2_hd64": lambda synth: synth.LMSpec("gpt2_hd64", "gpt2", 2, 128, 2, 2, 512, 300, 64, rand_affine=1),
    "qwen_hd64": lambda synth: synth.LMSpec("qwen_hd64", "qwen", 2, 256, 4, 2, 384, 411, 64, rope_theta=1e6, rand_affine=1),
    # weights rounded to bf16 in the file, opened with bf16_weights = 1: decode steps stream the exact 2-byte copies
    "qwen_hd64_bf16": lambda synth: synth.LMSpec("qwen_hd64_bf16", "qwen", 2, 256, 4, 2, 384, 411, 64, rope_theta=1e6, bf16_round=1),
    # the same two through the persistent cooperative decode kernel (rotary pairs, grouped heads, gated MLP)
    "gpt2_hd64_persistent": lambda synth: synth.LMSpec("gpt2_hd64", "gpt2", 2, 128, 2, 2, 512, 300, 64, rand_affine=1),
    "qwen_hd64_persistent": lambda synth: synth.LMSpec("qwen_hd64", "qwen", 2, 256, 4, 2, 384, 411, 64, rope_theta=1e6, rand_affine=1),
}


@pytest.mark.parametrize("kind", sorted(LM_SPECS))
def test_decoder_lm_logits_and_generation(cuda, tmp, kind):
    import orc
    import synth
    spec = LM_SPECS[kind](synth)
    cuda.ncmb_set_lm_persistent(int(kind.endswith("_persistent")))
    is_qwen = spec.kind == "qwen"
    conf, w = synth.write_lm(spec, tmp)
    cfg = cuda.load_config(conf)
    m = cuda.ncmb_lm_open(cfg, w.encode(), int(is_qwen), int(spec.bf16_round))
    assert m
    om = orc.LM(conf, w, is_qwen)
    prompts = synth.lm_prompts(spec, 3, 9, 3)
    for pr in prompts:
        pr = np.ascontiguousarray(pr)
        lg = np.zeros((pr.size, spec.vocab), np.float32)
        cuda.ncmb_lm_logits(m, pr.ctypes.data, pr.size, 0, lg.ctypes.data)
        _cmp_float(f"{kind} logits", lg, om.logits(pr), ATOL_LOGITS)
        last = np.zeros(spec.vocab, np.float32)
        cuda.ncmb_lm_logits(m, pr.ctypes.data, pr.size, 1, last.ctypes.data)
        _cmp_float(f"{kind} last logits", last, lg[-1], 1e-5)
    # batched KV-cache generation == independent full-recompute runs
    n_new = 12
    P = np.ascontiguousarray(prompts)
    for (t, tk, tp, sd) in ((0.0, 0, 1.0, 0), (0.9, 8, 1.0, 5), (0.7, 0, 0.95, 9)):
        out = np.zeros((P.shape[0], n_new), np.int32)
        cuda.ncmb_lm_generate(m, P.ctypes.data, P.shape[0], P.shape[1], n_new, t, tk, tp, sd, -1, out.ctypes.data)
        for b in range(P.shape[0]):
            want = om.generate(P[b], n_new, temp=t, top_k=tk, top_p=tp, seed=sd)
            assert (out[b] == want).all(), (kind, t, tk, tp, b, out[b], want)
        assert cuda.ncmb_gemm_tc_check() == 0           # no bounded wait (mbarrier, grid barrier) ran out
    cuda.ncmb_set_lm_persistent(0)
    cuda.ncmb_lm_close(m)


def _flush_c_stdout():
    import ctypes
    ctypes.CDLL(None).fflush(None)


PPL_SPECS = {
    # GPT-2 windows are n_ctx ids long (64 here); Qwen2 windows are 512 ids whatever the context length
    "gpt2": lambda synth: synth.LMSpec("gpt2_ppl", "gpt2", 2, 128, 2, 2, 512, 300, 64, rand_affine=1),
    "qwen": lambda synth: synth.LMSpec("qwen_ppl", "qwen", 2, 128, 2, 1, 256, 411, 600, rope_theta=1e6, rand_affine=1),
}


@pytest.mark.parametrize("decode_attention", ["chosen", "tensor_core_rows"])
@pytest.mark.parametrize("kind", ["gpt2", "qwen"])
def test_batched_decode_steps_through_k_sliced_projections(cuda, tmp, kind, decode_attention, monkeypatch):
    """20 rows per decode step at width 768: too many rows for the GEMV path, few tiles and a long K for the
    tensor-core GEMM, so the attention-output and MLP-down projections run K in slices with a reduce kernel behind
    them. Ids equal independent oracle runs. Run a second time with the decode attention that makes the (query, head)
    pairs of a kv group the rows of an mma.sync tile (what large batches of the grouped-query model get)."""
    import orc
    import synth
    if decode_attention == "tensor_core_rows":
        monkeypatch.setenv("NCM_B200_ATTN_DEC_MMA", "1")
    else:
        monkeypatch.delenv("NCM_B200_ATTN_DEC_MMA", raising=False)
    if kind == "gpt2":
        spec = synth.LMSpec("gpt2_w768", "gpt2", 1, 768, 12, 12, 3072, 300, 32, rand_affine=1)
    else:
        spec = synth.LMSpec("qwen_w768", "qwen", 1, 768, 12, 2, 2048, 300, 32, rope_theta=1e6, rand_affine=1)
    conf, w = synth.write_lm(spec, tmp)
    cfg = cuda.load_config(conf)
    m = cuda.ncmb_lm_open(cfg, w.encode(), int(kind == "qwen"), 0)
    om = orc.LM(conf, w, kind == "qwen")
    B, n_new = 20, 5
    P = np.ascontiguousarray(synth.lm_prompts(spec, B, 6, 17))
    out = np.zeros((B, n_new), np.int32)
    cuda.ncmb_lm_generate(m, P.ctypes.data, B, P.shape[1], n_new, 0.0, 0, 1.0, 0, -1, out.ctypes.data)
    for b in range(B):
        want = om.generate(P[b], n_new, temp=0.0)
        assert (out[b] == want).all(), (kind, b, out[b], want)
    assert cuda.ncmb_gemm_tc_check() == 0
    cuda.ncmb_lm_close(m)


@pytest.mark.parametrize("B", [2, 11])
def test_nucleus_sampling_over_a_vocabulary_too_large_for_the_block_sampler(cuda, tmp, B):
    """top_k = 0 over 2500 entries (the Qwen2 setting, temp 0.7 / top-p 0.95, at a size the oracle finishes quickly):
    every row's ids equal the oracle's full-sort walk."""
    import orc
    import synth
    spec = synth.LMSpec("qwen_v2500", "qwen", 1, 64, 2, 1, 128, 2500, 64, rope_theta=1e6, rand_affine=1)
    conf, w = synth.write_lm(spec, tmp)
    cfg = cuda.load_config(conf)
    m = cuda.ncmb_lm_open(cfg, w.encode(), 1, 0)
    om = orc.LM(conf, w, True)
    P = np.ascontiguousarray(synth.lm_prompts(spec, B, 7, 21))
    n_new = 10
    for (t, tp, sd) in ((0.7, 0.95, 9), (1.3, 0.5, 4)):
        out = np.zeros((B, n_new), np.int32)
        cuda.ncmb_lm_generate(m, P.ctypes.data, B, P.shape[1], n_new, t, 0, tp, sd, -1, out.ctypes.data)
        for b in range(B):
            want = om.generate(P[b], n_new, temp=t, top_k=0, top_p=tp, seed=sd)
            assert (out[b] == want).all(), (B, t, tp, b, out[b], want)
    cuda.ncmb_lm_close(m)


def test_nucleus_draw_by_selection_equals_the_sorted_walk(cuda, tmp):
    """The sort-free nucleus sampler (three-level descent over ordered keys with fixed-point probability mass) against
    the sort-based one and the oracle: a 5 000-entry vocabulary, 40 rows, several temperature / top-p settings, plus rows
    made of a few distinct logit values only, so that cuts and draws fall inside groups of tied entries."""
    import orc
    import synth
    spec = synth.LMSpec("qwen_v5000", "qwen", 1, 64, 2, 1, 128, 5000, 64, rope_theta=1e6, rand_affine=1)
    conf, w = synth.write_lm(spec, tmp)
    cfg = cuda.load_config(conf)
    m = cuda.ncmb_lm_open(cfg, w.encode(), 1, 0)
    om = orc.LM(conf, w, True)
    B, n_new = 40, 6
    P = np.ascontiguousarray(synth.lm_prompts(spec, B, 7, 33))
    try:
        for (t, tp, sd) in ((0.7, 0.95, 9), (1.3, 0.5, 4), (1.0, 1.0, 2), (0.2, 0.999, 7)):
            outs = {}
            for mode in ("1", "0"):
                os.environ["NCM_B200_SORT_SAMPLER"] = mode
                out = np.zeros((B, n_new), np.int32)
                cuda.ncmb_lm_generate(m, P.ctypes.data, B, P.shape[1], n_new, t, 0, tp, sd, -1, out.ctypes.data)
                outs[mode] = out
            assert np.array_equal(outs["0"], outs["1"]), (t, tp, np.argwhere(outs["0"] != outs["1"])[:5])
            for b in (0, 17, 39):
                want = om.generate(P[b], n_new, temp=t, top_k=0, top_p=tp, seed=sd)
                assert (outs["0"][b] == want).all(), (t, tp, b, outs["0"][b], want)
    finally:
        os.environ.pop("NCM_B200_SORT_SAMPLER", None)
    cuda.ncmb_lm_close(m)


def test_selection_sampler_on_rows_of_tied_logits(cuda):
    """Direct rows through sample_topkp's device twin: logits drawn from eight distinct values, so every key is held
    by hundreds of tied entries and both the nucleus cut and the draw land inside tie groups (ties rank by index)."""
    import ctypes as C
    import orc
    if not cuda.has("ncmb_sample_rows_dev"):
        pytest.skip("device row sampler not exported")
    rng = np.random.default_rng(12)
    V, B = 6000, 24
    vals = np.array([-3.0, -1.5, -0.25, 0.0, 0.5, 1.0, 2.0, 2.5], np.float32)
    lg = vals[rng.integers(0, 8, size=(B, V))]
    lg[3] = 1.25                                            # one constant row: a single key for the whole vocabulary
    u = rng.random(B)
    d_lg, d_u, d_out = cuda.to_backend(lg), cuda.to_backend(u.astype(np.float64)), cuda.alloc(B)
    for (t, tp) in ((0.8, 0.9), (1.0, 0.35), (2.0, 1.0)):
        got = {}
        for mode in ("1", "0"):
            os.environ["NCM_B200_SORT_SAMPLER"] = mode
            cuda.ncmb_sample_rows_dev(d_lg, B, V, t, 0, tp, d_u, d_out)
            got[mode] = cuda.to_host(d_out, (B,), np.int32)
        os.environ.pop("NCM_B200_SORT_SAMPLER", None)
        assert np.array_equal(got["0"], got["1"]), (t, tp, got)
        for b in range(B):
            # the oracle's walk with the same uniform: a stable descending order (ties by ascending index)
            w_ = (lg[b] / np.float32(t)).astype(np.float32)
            order = np.argsort(-w_.astype(np.float64), kind="stable")
            p = np.exp(w_[order].astype(np.float64) - float(w_[order[0]]))
            p /= p.sum()
            cum, nkeep = 0.0, V
            for r in range(V):
                if cum - p[r] > tp:
                    nkeep = r
                    break
                cum += p[r]
            den = p[:nkeep].sum()
            acc, pick = 0.0, order[nkeep - 1]
            x = u[b] * den
            c = np.cumsum(p[:nkeep])
            j = int(np.searchsorted(c, x, side="left"))
            pick = order[min(j, nkeep - 1)]
            assert got["0"][b] == pick, (t, tp, b, got["0"][b], pick)


@pytest.mark.parametrize("kind", sorted(PPL_SPECS))
def test_decoder_lm_likelihood_and_fixture_commands(cuda, tmp, kind, capfd):
    """ncmb_lm_nll, *_cmd_ppl and *_cmd_verify against the oracle's window likelihood (reference gpt2_nll / qwen_nll)."""
    import orc
    import synth
    spec = PPL_SPECS[kind](synth)
    is_qwen = kind == "qwen"
    conf, w = synth.write_lm(spec, tmp)
    cfg = cuda.load_config(conf)
    om = orc.LM(conf, w, is_qwen)
    window = 512 if is_qwen else spec.n_ctx
    docs = [synth.lm_prompts(spec, 1, n, 11 + i)[0] for i, n in enumerate((9, 2 * window + 22, 33, window + 1, 1))]
    # the windows the reference cuts (gpt2.c:253-260, qwen.c:283-288) and their likelihoods from the oracle
    wins = []
    for d in docs:
        if d.size < 2:
            continue
        o = 0
        while o + 1 < d.size:
            T = min(window, d.size - o)
            if T < 2:
                break
            wins.append(d[o:o + T])
            o += window
    want = np.array([om.nll(x) for x in wins])
    tol = 5e-5                                # logits agree to about 1e-5; the likelihood is a smooth function of them
    m = cuda.ncmb_lm_open(cfg, w.encode(), int(is_qwen), 0)
    # one window at a time, then all of them ragged in one batch
    one = np.zeros(len(wins))
    for i, x in enumerate(wins):
        x = np.ascontiguousarray(x, np.int32)
        got = np.zeros(1)
        cuda.ncmb_lm_nll(m, x.ctypes.data, 1, x.size, None, got.ctypes.data)
        one[i] = got[0]
    assert np.abs(one - want).max() < tol, (one, want)
    T = max(x.size for x in wins)
    ids = np.full((len(wins), T), 7, np.int32)            # tail padding must not matter
    lens = np.array([x.size for x in wins], np.int32)
    for i, x in enumerate(wins):
        ids[i, :x.size] = x
    got = np.zeros(len(wins))
    cuda.ncmb_lm_nll(m, ids.ctypes.data, len(wins), T, lens.ctypes.data, got.ctypes.data)
    assert np.abs(got - want).max() < tol, (got, want)
    cuda.ncmb_lm_close(m)

    # *_cmd_ppl: ids per line (no host tokenizer is linked into the test process)
    texts = os.path.join(tmp, f"{kind}_texts.txt")
    with open(texts, "w") as f:
        for d in docs:
            f.write(" ".join(str(int(v)) for v in d) + "\n\n")
    capfd.readouterr()
    rc = getattr(cuda, f"{kind if is_qwen else 'gpt2'}_cmd_ppl")(cfg, w.encode(), tmp.encode(), texts.encode())
    _flush_c_stdout()
    line = [ln for ln in capfd.readouterr().out.splitlines() if ln.startswith("docs=")][-1]
    assert rc == 0
    ntok = sum(x.size - 1 for x in wins)
    tot = 0.0
    for x, v in zip(wins, want):
        tot += v * (x.size - 1)
    f = dict(kv.split("=") for kv in line.split())
    assert int(f["docs"]) == sum(1 for d in docs if d.size >= 2) and int(f["tokens"]) == ntok, line
    assert abs(float(f["nll"]) - tot / ntok) < 1e-4 and abs(float(f["ppl"]) - np.exp(tot / ntok)) < 1e-4 * np.exp(tot / ntok) + 1e-5, line

    # *_cmd_verify on fixtures written from the oracle: logits pass, a disturbed file fails
    fx = os.path.join(tmp, f"{kind}_fx")
    os.makedirs(fx, exist_ok=True)
    names = {"s1": docs[0], "s2": docs[2]}
    with open(os.path.join(fx, f"{kind}_tok.txt"), "w") as f:
        for nm, d in names.items():
            f.write(f"{nm}\t{'text'.encode().hex()}\t{' '.join(str(int(v)) for v in d)}\n")
            om.logits(d).tofile(os.path.join(fx, f"{kind}_logits_{nm}.f32"))
    with open(os.path.join(fx, f"{kind}_gen.txt"), "w") as f:
        f.write(f"g1\t{'text'.encode().hex()}\t1 2 3\n")
    with open(os.path.join(fx, f"{kind}_ppl.txt"), "w") as f:
        f.write(f"{'text'.encode().hex()}\t{want[0]:.6f}\t{np.exp(want[0]):.4f}\n")
    verify = getattr(cuda, f"{kind}_cmd_verify")
    rc = verify(cfg, w.encode(), tmp.encode(), fx.encode())
    _flush_c_stdout()
    out = capfd.readouterr().out
    assert rc == 0, out
    assert out.count("ok   logits") == 2 and f"{kind.upper()}-VERIFY PASS (6 checked)" in out, out
    bad = om.logits(names["s2"])
    bad[3, 5] += 0.5
    bad.tofile(os.path.join(fx, f"{kind}_logits_s2.f32"))
    rc = verify(cfg, w.encode(), tmp.encode(), fx.encode())
    _flush_c_stdout()
    out = capfd.readouterr().out
    assert rc == 1 and "FAIL logits s2" in out and f"{kind.upper()}-VERIFY FAIL" in out, out


def test_training_checkpoints_load_as_weights(cuda, tmp, capfd):
    """weights_load on an NCK1 training checkpoint (reference src/tensor.c:73-80 -> ckpt_load_weights_only
    src/ckpt.c:549-625): same tensors as the NCM1 file, checksum and truncation are refused, and a model opened
    from the checkpoint computes what it computes from the weights file."""
    import ctypes as C
    import synth
    spec = synth.spec_gpt2_tiny()
    conf, w = synth.write_lm(spec, tmp)
    tensors = synth.lm_tensors(spec, 1)
    ncm = os.path.join(tmp, "ck_same.ncm")
    ck = os.path.join(tmp, "ck_same.nckpt")
    synth.write_ncm(ncm, tensors)
    synth.write_nck1(ck, tensors, optimizer_slots=2)
    assert cuda.ckpt_probe(ck.encode()) == 1 and cuda.ckpt_probe(ncm.encode()) == 0
    assert cuda.ckpt_probe(conf.encode()) == -1 and cuda.ckpt_probe(b"/nonexistent/file") == -1
    a, b = cuda.load_weights(ncm), cuda.load_weights(ck)
    assert a.count == b.count == len(tensors)
    for name, want in tensors.items():
        got = cuda.tensor_host(b, name)
        assert helpers.same_bits(got, np.ascontiguousarray(want, np.float32)), name
        assert helpers.same_bits(got, cuda.tensor_host(a, name)), name
    cuda.weights_free(C.byref(a))
    cuda.weights_free(C.byref(b))
    # refusals: a flipped byte (checksum), a cut file, a wrong version
    raw = open(ck, "rb").read()
    import struct
    variants = {"flip": raw[:len(raw) // 2] + bytes([raw[len(raw) // 2] ^ 1]) + raw[len(raw) // 2 + 1:],
                "cut": raw[:len(raw) // 3]}
    v2 = bytearray(raw[:-8])
    v2[4:8] = struct.pack("<I", 2)
    variants["version"] = bytes(v2) + struct.pack("<Q", synth._fnv1a64(bytes(v2)))
    for tag, data in variants.items():
        path = os.path.join(tmp, f"ck_{tag}.nckpt")
        open(path, "wb").write(data)
        import capi
        ws = capi.WeightStore()
        err = C.create_string_buffer(256)
        assert cuda.ckpt_load_weights_only(path.encode(), C.byref(ws), err, 256) == -1, tag
        assert ws.count == 0 and not ws.items
        msg = err.value.decode()
        assert ("checksum mismatch" in msg) if tag != "version" else ("not an NCK1 checkpoint" in msg), (tag, msg)
        assert cuda.weights_load(C.byref(ws), path.encode()) == -1
    capfd.readouterr()
    # a decoder LM opened straight from a checkpoint of its weights
    ck2 = os.path.join(tmp, "lm_from_ckpt.nckpt")
    synth.write_nck1(ck2, _read_ncm(w))
    cfg = cuda.load_config(conf)
    pr = np.ascontiguousarray(synth.lm_prompts(spec, 1, 9, 3)[0])
    outs = []
    for path in (w, ck2):
        m = cuda.ncmb_lm_open(cfg, path.encode(), 0, 0)
        assert m
        lg = np.zeros((pr.size, spec.vocab), np.float32)
        cuda.ncmb_lm_logits(m, pr.ctypes.data, pr.size, 0, lg.ctypes.data)
        outs.append(lg)
        cuda.ncmb_lm_close(m)
    assert helpers.same_bits(outs[0], outs[1])


def _read_ncm(path):
    """tensors of an NCM1 file, in file order"""
    import struct
    out = {}
    with open(path, "rb") as f:
        assert f.read(4) == b"NCM1"
        (count,) = struct.unpack("<I", f.read(4))
        for _ in range(count):
            (nl,) = struct.unpack("<B", f.read(1))
            name = f.read(nl).decode()
            (nd,) = struct.unpack("<B", f.read(1))
            shape = struct.unpack(f"<{nd}I", f.read(4 * nd))
            (nb,) = struct.unpack("<Q", f.read(8))
            out[name] = np.frombuffer(f.read(nb), np.float32).reshape(shape).copy()
    return out


@pytest.mark.parametrize("kind", ["gpt2", "qwen"])
def test_safetensors_import_on_the_device(cuda, tmp, kind):
    """ncmb_weights_import_safetensors against the converters' rules (orc.safetensors_import_rules, itself pinned
    against tools/gpt2import.c / tools/qwenimport.c in the CPU suite), and a model opened from the checkpoint."""
    import ctypes as C
    import capi
    import orc
    import synth
    from test_oracle_pin import _hf_files
    spec, paths = _hf_files(tmp, kind)
    for tag, p in paths.items():
        want = orc.safetensors_import_rules(p, kind == "gpt2")
        ws = capi.WeightStore()
        assert cuda.ncmb_weights_import_safetensors(C.byref(ws), p.encode(), int(kind == "gpt2")) == 0
        assert ws.count == len(want)
        for name, w in want.items():
            got = cuda.tensor_host(ws, name)
            assert got is not None and helpers.same_bits(got, w), (tag, name)
        assert cuda.tensor_host(ws, "h.0.attn.bias") is None
        cuda.weights_free(C.byref(ws))
    # broken files are refused
    raw = open(paths["f32"], "rb").read()
    for tag, data in (("cut", raw[:len(raw) // 2]), ("nojson", raw[:8] + b"[" + raw[9:])):
        bad = os.path.join(tmp, f"{kind}_{tag}.safetensors")
        open(bad, "wb").write(data)
        ws = capi.WeightStore()
        assert cuda.ncmb_weights_import_safetensors(C.byref(ws), bad.encode(), 1) == -1, tag
        assert ws.count == 0 and not ws.items
    # the model runs from the checkpoint as it runs from the converted weights
    conf, w = synth.write_lm(spec, tmp)
    cfg = cuda.load_config(conf)
    pr = np.ascontiguousarray(synth.lm_prompts(spec, 1, 9, 3)[0])
    outs = []
    for path in (w, paths["f32"]):
        m = cuda.ncmb_lm_open(cfg, path.encode(), int(kind == "qwen"), 0)
        assert m
        lg = np.zeros((pr.size, spec.vocab), np.float32)
        cuda.ncmb_lm_logits(m, pr.ctypes.data, pr.size, 0, lg.ctypes.data)
        outs.append(lg)
        cuda.ncmb_lm_close(m)
    assert helpers.same_bits(outs[0], outs[1])


def test_two_byte_weight_file_variant(cuda, tmp):
    """"NCM2" files (bf16 records widened on the device): same tensors as the fp32 file of the same values, a decoder
    opened from one streams 2-byte copies without being told and computes what it computes from the fp32 file;
    malformed records are refused."""
    import ctypes as C
    import struct
    import capi
    import orc
    import synth
    spec = synth.LMSpec("qwen_ncm2", "qwen", 2, 256, 4, 2, 384, 411, 64, rope_theta=1e6, bf16_round=1)
    conf, w1 = synth.write_lm(spec, tmp)
    tensors = synth.lm_tensors(spec, 4321)
    w2 = os.path.join(tmp, "qwen_ncm2.ncm2")
    synth.write_ncm2(w2, tensors)
    assert os.path.getsize(w2) < 0.55 * os.path.getsize(w1)
    a, b = cuda.load_weights(w1), cuda.load_weights(w2)
    assert a.count == b.count == len(tensors)
    assert cuda.ncmb_weights_are_bf16(C.byref(a)) == 0 and cuda.ncmb_weights_are_bf16(C.byref(b)) == 1
    for name, want in tensors.items():
        assert helpers.same_bits(cuda.tensor_host(b, name), np.ascontiguousarray(want, np.float32)), name
    cuda.weights_free(C.byref(a))
    cuda.weights_free(C.byref(b))
    cfg = cuda.load_config(conf)
    om = orc.LM(conf, w1, True)
    P = np.ascontiguousarray(synth.lm_prompts(spec, 3, 9, 3))
    outs = []
    for path, flag in ((w1, 1), (w2, 0)):
        m = cuda.ncmb_lm_open(cfg, path.encode(), 1, flag)
        assert m
        lg = np.zeros((P.shape[1], spec.vocab), np.float32)
        cuda.ncmb_lm_logits(m, P[0].ctypes.data, P.shape[1], 0, lg.ctypes.data)
        ids = np.zeros((3, 10), np.int32)
        cuda.ncmb_lm_generate(m, P.ctypes.data, 3, P.shape[1], 10, 0.0, 0, 1.0, 0, -1, ids.ctypes.data)
        outs.append((lg, ids))
        cuda.ncmb_lm_close(m)
    assert helpers.same_bits(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    _cmp_float("ncm2 logits", outs[1][0], om.logits(P[0]), ATOL_LOGITS)
    for b_ in range(3):
        assert (outs[1][1][b_] == om.generate(P[b_], 10, temp=0.0)).all()
    # refusals: an element type the loader does not know, a payload that does not match the shape, a cut file
    raw = bytearray(open(w2, "rb").read())
    name0 = next(iter(tensors))
    tpos = 8 + 1 + len(name0.encode()) + 1 + 4 * tensors[name0].ndim
    assert raw[tpos] == 1
    bad = {"type": bytes(raw[:tpos]) + b"\x07" + bytes(raw[tpos + 1:]),
           "size": bytes(raw[:tpos]) + b"\x00" + bytes(raw[tpos + 1:]),          # 2-byte payload declared as fp32
           "cut": bytes(raw[:len(raw) // 2]),
           "count": bytes(raw[:4]) + struct.pack("<I", 0xFFFFFFF0) + bytes(raw[8:])}
    for tag, data in bad.items():
        path = os.path.join(tmp, f"bad_{tag}.ncm2")
        open(path, "wb").write(data)
        ws = capi.WeightStore()
        assert cuda.weights_load(C.byref(ws), path.encode()) == -1, tag
        assert ws.count == 0 and not ws.items


def test_rewriting_a_weight_tensor_drops_its_cached_copies(cuda, tmp):
    """The GEMM engines cache converted copies of weight matrices by device address. A matrix rewritten in place with
    tensor_to_backend must run on its new values, like a model loaded from a file with those values."""
    import ctypes as C
    import capi
    import cases
    import synth
    spec = cases.ncp_spec("plain")
    conf, w = synth.write_ncp(spec, tmp)
    pre, l0, _ = cases.ncp_inputs(spec)
    m = capi.NcpModel(cuda, conf, w, arena_mb=64)
    before = m.generate(pre, temp=0.0)
    tens = synth.ncp_tensors(spec, 1234)
    name = "gen.transformer.blocks.0.mlp.c_fc.weight"     # a prefix-pass projection: 36 token rows, tensor-core engine, cached pairs
    new = np.ascontiguousarray(np.random.default_rng(1).normal(0, 0.02, tens[name].shape), np.float32)
    t = cuda.weights_get(C.byref(m.ws), name.encode())
    assert t
    tb = cuda.lib.tensor_to_backend
    tb.restype, tb.argtypes = None, [C.c_void_p, C.c_void_p]
    tb(t, new.ctypes.data)
    after = m.generate(pre, temp=0.0)
    tens[name] = new
    w2 = os.path.join(tmp, "plain_rewritten.ncm")
    synth.write_ncm(w2, tens)
    fresh = capi.NcpModel(cuda, conf, w2, arena_mb=64).generate(pre, temp=0.0)
    assert np.array_equal(after, fresh)
    assert not np.array_equal(after, before)
