"""Case runners shared by the golden generator and the parity tests.

``capi_*`` drive any library exporting the reference's C interface (the
reference CPU build, or libncm_b200.so on a GPU) through ctypes;
``orc_*`` drive the CPU oracle.  Both fill a dict with the same keys, which is
what tests compare against each other and against tests/golden/golden.npz.
"""
import ctypes as C
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for _p in (os.path.join(ROOT, "saphira-cncm_b200"), os.path.join(ROOT, "oracle"),
           os.path.join(HERE, "golden"), HERE):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import capi      # noqa: E402
import cases     # noqa: E402
import synth     # noqa: E402

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libcncm_ref.so")
CUDA_LIB = os.path.join(ROOT, "saphira-cncm_b200", "libncm_b200.so")
GOLDEN = os.path.join(HERE, "golden", "golden.npz")


def sha(path):
    return hashlib.sha256(open(path, "rb").read()).hexdigest()


def capi_kernels(ref, out):
    d = cases.kernel_inputs()
    B = ref.to_backend
    H = ref.to_host

    # linear
    for tag, x, W, b in (("lin", d["lin_x"], d["lin_W"], d["lin_b"]), ("lin2", d["lin2_x"], d["lin2_W"], None)):
        y = ref.alloc(x.shape[0] * W.shape[0])
        ref.linear_fwd(B(x), B(W), B(b) if b is not None else None, y, x.shape[0], W.shape[0], W.shape[1])
        out["k_" + tag] = H(y, (x.shape[0], W.shape[0]))
    x, w, b = d["ln_x"], d["ln_w"], d["ln_b"]
    y = ref.alloc(x.size)
    ref.layernorm_fwd(B(x), B(w), B(b), y, 4, 64); out["k_ln"] = H(y, x.shape)
    ref.layernorm_fwd(B(x), B(w), None, y, 4, 64); out["k_ln_nob"] = H(y, x.shape)
    ref.layernorm_eps_fwd(B(x), B(w), B(b), y, 4, 64, 1e-5); out["k_ln_eps"] = H(y, x.shape)
    ref.rmsnorm_fwd(B(x), B(w), y, 4, 64); out["k_rms"] = H(y, x.shape)
    a = d["act_x"]
    y = ref.alloc(a.size)
    for nm in ("gelu", "gelu_tanh", "silu"):
        getattr(ref, nm + "_fwd")(B(a), y, a.size); out["k_" + nm] = H(y, a.shape)
    ref.softmax_fwd(B(a), y, 8, 64); out["k_softmax"] = H(y, (8, 64))
    q, k = B(d["rope_q"]), B(d["rope_k"])
    ref.rope_apply(q, k, B(d["rope_cos"]), B(d["rope_sin"]), 1, 2, 16, 32)
    out["k_rope_q"], out["k_rope_k"] = H(q, d["rope_q"].shape), H(k, d["rope_k"].shape)
    ref.arena_init(64 << 20)
    o = ref.alloc(d["sd_q"].size)
    ref.sdpa_fwd(B(d["sd_q"]), B(d["sd_k"]), B(d["sd_v"]), B(d["sd_mask"]), o, 1, 2, 8, 12, 16)
    out["k_sdpa"] = H(o, d["sd_q"].shape)
    o = ref.alloc(d["gq_q"].size)
    ref.sdpa_fwd_gqa(B(d["gq_q"]), B(d["gq_k"]), B(d["gq_v"]), None, o, 2, 4, 2, 5, 7, 8)
    out["k_sdpa_gqa"] = H(o, d["gq_q"].shape)
    x = d["cv_x"]
    y = ref.alloc(x.size)
    ref.conv1d_fwd(B(x), B(d["cv_W"]), B(d["cv_b"]), y, 2, 4, 4, 32, 3, 1, 1); out["k_conv"] = H(y, x.shape)
    ref.conv1d_fwd(B(x), B(d["cs_W"]), B(d["cv_b"]), y, 2, 4, 4, 32, 2, 2, 0); out["k_conv_s2"] = H(y, (2, 4, 16))
    y2 = ref.alloc(2 * 4 * 64)
    ref.convtranspose1d_fwd(B(x), B(d["cs_W"]), B(d["cv_b"]), y2, 2, 4, 4, 32, 2, 2); out["k_convT"] = H(y2, (2, 4, 64))
    ref.groupnorm_fwd(B(x), y, 2, 2, 4, 32); out["k_gn"] = H(y, x.shape)
    ref.interpolate_area_fwd(B(d["ar_x"]), y, 2, 4, 32, 9); out["k_area"] = H(y, (2, 4, 9))
    ref.interpolate_area_fwd(B(d["ar_x"]), y, 2, 4, 32, 1); out["k_area1"] = H(y, (2, 4, 1))
    ref.interpolate_linear_fwd(B(d["li_x"]), y, 2, 4, 9, 32); out["k_lin_interp"] = H(y, (2, 4, 32))
    ref.interpolate_linear_fwd(B(d["li_x"][:, :, :1].copy()), y, 2, 4, 1, 8); out["k_lin_interp1"] = H(y, (2, 4, 8))
    dd = ref.alloc(16 * 8)
    ref.rowwise_l2sq(B(d["l2_a"]), B(d["l2_b"]), dd, 16, 8, 32); out["k_l2sq"] = H(dd, (16, 8))
    # data movement and element-wise kernels (src/ncm.h:149, 161-165, 184-190)
    W, idx = d["emb_W"], d["emb_idx"]
    y = ref.alloc(idx.size * W.shape[1])
    ref.embedding_fwd(B(W), B(idx), y, idx.size, W.shape[1]); out["k_embedding"] = H(y, (idx.size, W.shape[1]))
    q, k = B(d["rg_q"]), B(d["rg_k"])
    ref.rope_apply_gqa(q, k, B(d["rg_cos"]), B(d["rg_sin"]), 2, 6, 2, 5, 16)
    out["k_rope_gqa_q"], out["k_rope_gqa_k"] = H(q, d["rg_q"].shape), H(k, d["rg_k"].shape)
    y = ref.alloc(d["htb_x"].size)
    ref.heads_transpose_fwd(B(d["ht_x"]), y, 7, 3, 8); out["k_heads_t"] = H(y, (3, 7, 8))
    ref.heads_transpose_fwd_b(B(d["htb_x"]), y, 2, 7, 3, 8); out["k_heads_tb"] = H(y, (2, 3, 7, 8))
    a, b = d["ew_a"], d["ew_b"]
    y = ref.alloc(a.size)
    ref.add_fwd(B(a), B(b), y, a.size); out["k_add"] = H(y, a.shape)
    ref.mul_fwd(B(a), B(b), y, a.size); out["k_mul"] = H(y, a.shape)
    ref.scale_fwd(B(a), 0.37, y, a.size); out["k_scale"] = H(y, a.shape)
    acc = B(a)
    ref.add_inplace_fwd(acc, B(b), a.size); out["k_add_inplace"] = H(acc, a.shape)
    s = cases.QS
    n = s["B"] * s["H"] * s["T"] * s["hd"]
    qq, kk, vv = ref.alloc(n), ref.alloc(n), ref.alloc(n)
    ref.qkv_split_fwd(B(d["qs_x"]), qq, kk, vv, s["B"], s["T"], s["C"], s["H"], s["hd"], s["K"], s["rep"])
    shp = (s["B"], s["H"], s["T"], s["hd"])
    out["k_qkv_q"], out["k_qkv_k"], out["k_qkv_v"] = H(qq, shp), H(kk, shp), H(vv, shp)
    s = cases.HM
    y = ref.alloc(s["B"] * s["T"] * s["C"])
    ref.head_merge_fwd(B(d["hm_x"]), y, s["B"], s["T"], s["C"], s["H"], s["hd"])
    out["k_head_merge"] = H(y, (s["B"], s["T"], s["C"]))
    # sampling: one shared stream across six rows and three settings
    picks = []
    st = C.c_ulonglong(0x1234ABCD)
    for (t, tk, tp) in ((0.0, 0, 1.0), (0.8, 5, 0.9), (1.0, 0, 0.6), (0.7, 50, 1.0)):
        for r in range(d["smp"].shape[0]):
            row = np.ascontiguousarray(d["smp"][r])
            picks.append(ref.sample_topkp(row.ctypes.data, row.size, t, tk, tp, C.byref(st)))
    out["k_sample"] = np.array(picks, np.int32)
    out["k_sample_state"] = np.array([st.value], np.uint64)
    st = C.c_ulonglong(42)
    out["k_rng"] = np.array([ref.rng_next(C.byref(st)) for _ in range(8)], np.uint64)


def capi_ncp(ref, out, tmp, variants=None, with_c1=True):
    for var in (variants or cases.NCP_VARIANTS):
        spec = cases.ncp_spec(var)
        conf, w = synth.write_ncp(spec, tmp)
        out[f"sha_{var}"] = np.frombuffer(bytes.fromhex(sha(w)), np.uint8)
        m = capi.NcpModel(ref, conf, w, arena_mb=256)
        pre, l0, ids = cases.ncp_inputs(spec)
        B = pre.shape[0]
        for sname in cases.SAMPLERS:
            kw = cases.sampler_kwargs(sname, spec)
            if kw.get("cfg", 0) > 0 and spec.pad_id < 0:
                continue                                   # CFG needs pad/eos ids
            use_l0 = l0 if not spec.query_level0 else None
            out[f"codes_{var}_{sname}"] = m.generate(pre, l0=use_l0, **kw)
        if spec.query_level0:
            out[f"codes_{var}_l0given"] = m.generate(pre, l0=l0, temp=0.0)
        # quantizer + VQ-VAE stages (the reference's `infer` walk, src/main.c:243-268)
        D, L, nl = spec.vq_dim, spec.L, len(spec.levels)
        ref.arena_reset()
        z = ref.alloc(B * L * D)
        ref.vqvae_encode_z(m.vqvae, ids.ctypes.data, z, B)
        out[f"encz_{var}"] = ref.to_host(z, (B, L, D))
        idx = np.zeros((B, m.total), np.int32)
        ref.vq_z_to_idx(m.vq, z, B, idx.ctypes.data)
        out[f"idx_{var}"] = idx
        zh = [ref.alloc(B * L * D) for _ in range(nl)]
        arr = (C.c_void_p * nl)(*zh)
        ref.arena_reset()
        ref.vq_idx_to_zhats(m.vq, idx.ctypes.data, B, arr)
        out[f"zhats_{var}"] = np.stack([ref.to_host(p, (B, L, D)) for p in zh])
        lg = ref.alloc(B * L * spec.in_vocab)
        ref.arena_reset()
        ref.vqvae_decode(m.vqvae, zh[-1], lg, B)
        out[f"declogits_{var}"] = ref.to_host(lg, (B, L, spec.in_vocab))
        # teacher-forced forward
        lvl_first = 0 if spec.query_level0 else 1
        T2 = m.total - spec.levels[0]
        xin = ref.alloc(B * T2 * D)
        ref.arena_reset()
        ref.vq_idx_to_ncm_input(m.vq, idx.ctypes.data, B, xin)
        out[f"ncminput_{var}"] = ref.to_host(xin, (B, T2, D))
        T = m.total - (spec.levels[0] if lvl_first else 0)
        P = spec.prefix_len
        # x = [wte(prefix) ; (l0 queries) ; ncm input]
        tens = synth.ncp_tensors(spec, 1234)
        zpre = tens["tok.encoder.wte.weight"][pre]                     # [B,P,D]
        parts = [zpre]
        if spec.query_level0:
            parts.append(np.broadcast_to(tens["gen.l0_queries"].reshape(1, spec.levels[0], D),
                                         (B, spec.levels[0], D)))
        parts.append(out[f"ncminput_{var}"])
        x = np.ascontiguousarray(np.concatenate(parts, axis=1), dtype=np.float32)
        assert x.shape[1] == P + T, (x.shape, P, T)
        maxV = max(spec.vocab[lvl_first:])
        lgd = ref.alloc(B * T * maxV)
        ref.arena_reset()
        ref.ncp_forward(m.ncp, ref.to_backend(x), pre.ctypes.data, lgd, B)
        out[f"fwdlogits_{var}"] = ref.to_host(lgd, (B, T, maxV))
    # the PR1-shaped small model, 4 rows
    for ladder, nm in () if not with_c1 else (((1, 3, 9), "c1"), ((1, 3, 9, 81), "c1b")):
        spec = synth.spec_c1(ladder)
        conf, w = synth.write_ncp(spec, tmp)
        out[f"sha_{nm}"] = np.frombuffer(bytes.fromhex(sha(w)), np.uint8)
        m = capi.NcpModel(ref, conf, w, arena_mb=1024)
        pre = synth.ncp_prefixes(spec, 4, 7)
        out[f"codes_{nm}_greedy"] = m.generate(pre, temp=0.0)
        out[f"codes_{nm}_topk"] = m.generate(pre, temp=0.8, top_k=50, top_p=0.9, seed=3)




# ---------------------------------------------------------------------------
# the same cases through the CPU oracle
# ---------------------------------------------------------------------------

def orc_kernels(out):
    import orc
    d = cases.kernel_inputs()
    out["k_lin"] = orc.linear(d["lin_x"], d["lin_W"], d["lin_b"])
    out["k_lin2"] = orc.linear(d["lin2_x"], d["lin2_W"], None)
    out["k_ln"] = orc.layernorm(d["ln_x"], d["ln_w"], d["ln_b"])
    out["k_ln_nob"] = orc.layernorm(d["ln_x"], d["ln_w"], None)
    out["k_ln_eps"] = orc.layernorm(d["ln_x"], d["ln_w"], d["ln_b"], eps=float(np.float32(1e-5)))
    out["k_rms"] = orc.rmsnorm(d["ln_x"], d["ln_w"])
    out["k_gelu"], out["k_gelu_tanh"], out["k_silu"] = orc.gelu(d["act_x"]), orc.gelu_tanh(d["act_x"]), orc.silu(d["act_x"])
    out["k_softmax"] = orc.softmax(d["act_x"].reshape(8, 64))
    out["k_rope_q"] = orc.rope(d["rope_q"], d["rope_cos"], d["rope_sin"], 16)
    out["k_rope_k"] = orc.rope(d["rope_k"], d["rope_cos"], d["rope_sin"], 16)
    out["k_sdpa"] = orc.sdpa(d["sd_q"], d["sd_k"], d["sd_v"], d["sd_mask"])
    out["k_sdpa_gqa"] = orc.sdpa(d["gq_q"], d["gq_k"], d["gq_v"], None)
    out["k_conv"] = orc.conv1d(d["cv_x"], d["cv_W"], d["cv_b"], 1, 1)
    out["k_conv_s2"] = orc.conv1d(d["cv_x"], d["cs_W"], d["cv_b"], 2, 0)
    out["k_convT"] = orc.convT1d(d["cv_x"], d["cs_W"], d["cv_b"], 2)
    out["k_gn"] = orc.groupnorm(d["cv_x"], 2)
    out["k_area"], out["k_area1"] = orc.interp_area(d["ar_x"], 9), orc.interp_area(d["ar_x"], 1)
    out["k_lin_interp"] = orc.interp_linear(d["li_x"], 32)
    out["k_lin_interp1"] = orc.interp_linear(d["li_x"][:, :, :1].copy(), 8)
    out["k_l2sq"] = orc.l2sq(d["l2_a"], d["l2_b"])
    out["k_embedding"] = orc.embedding(d["emb_W"], d["emb_idx"])
    out["k_rope_gqa_q"], out["k_rope_gqa_k"] = orc.rope_gqa(d["rg_q"], d["rg_k"], d["rg_cos"], d["rg_sin"])
    out["k_heads_t"] = orc.heads_transpose(d["ht_x"], 7, 3, 8)
    out["k_heads_tb"] = orc.heads_transpose_b(d["htb_x"], 2, 7, 3, 8)
    out["k_add"], out["k_mul"] = orc.add(d["ew_a"], d["ew_b"]), orc.mul(d["ew_a"], d["ew_b"])
    out["k_scale"] = orc.scale(d["ew_a"], 0.37)
    out["k_add_inplace"] = orc.add(d["ew_a"], d["ew_b"])
    s = cases.QS
    out["k_qkv_q"], out["k_qkv_k"], out["k_qkv_v"] = orc.qkv_split(d["qs_x"], s["B"], s["T"], s["C"], s["H"], s["hd"], s["K"], s["rep"])
    s = cases.HM
    out["k_head_merge"] = orc.head_merge(d["hm_x"], s["B"], s["T"], s["C"], s["H"], s["hd"])
    picks, st = [], 0x1234ABCD
    for (t, tk, tp) in ((0.0, 0, 1.0), (0.8, 5, 0.9), (1.0, 0, 0.6), (0.7, 50, 1.0)):
        for r in range(d["smp"].shape[0]):
            p, st = orc.sample_topkp(d["smp"][r], t, tk, tp, st)
            picks.append(p)
    out["k_sample"] = np.array(picks, np.int32)
    out["k_sample_state"] = np.array([st], np.uint64)
    s = C.c_uint64(42)
    out["k_rng"] = np.array([orc.lib().orc_rng_next(C.byref(s)) for _ in range(8)], np.uint64)


def orc_ncp(out, tmp, variants=None, with_c1=True):
    import orc
    for var in (variants or cases.NCP_VARIANTS):
        spec = cases.ncp_spec(var)
        conf, w = synth.write_ncp(spec, tmp)
        out[f"sha_{var}"] = np.frombuffer(bytes.fromhex(sha(w)), np.uint8)
        m = orc.Model(conf, w)
        pre, l0, ids = cases.ncp_inputs(spec)
        B = pre.shape[0]
        for sname in cases.SAMPLERS:
            kw = cases.sampler_kwargs(sname, spec)
            if kw.get("cfg", 0) > 0 and spec.pad_id < 0:
                continue
            use_l0 = l0 if not spec.query_level0 else None
            out[f"codes_{var}_{sname}"] = m.generate(pre, l0=use_l0, **kw)
        if spec.query_level0:
            out[f"codes_{var}_l0given"] = m.generate(pre, l0=l0, temp=0.0)
        nl, D = len(spec.levels), spec.vq_dim
        z = m.encode(ids)
        out[f"encz_{var}"] = z
        idx = m.z_to_idx(z)
        out[f"idx_{var}"] = idx
        zh = m.idx_to_zhats(idx, nl)
        out[f"zhats_{var}"] = np.stack(zh)
        out[f"declogits_{var}"] = m.decode(zh[-1])
        T2 = m.total - spec.levels[0]
        xin = m.idx_to_ncm_input(idx, T2)
        out[f"ncminput_{var}"] = xin
        tens = synth.ncp_tensors(spec, 1234)
        parts = [tens["tok.encoder.wte.weight"][pre]]
        if spec.query_level0:
            parts.append(np.broadcast_to(tens["gen.l0_queries"].reshape(1, spec.levels[0], D),
                                         (B, spec.levels[0], D)))
        parts.append(xin)
        x = np.ascontiguousarray(np.concatenate(parts, axis=1), dtype=np.float32)
        out[f"fwdlogits_{var}"] = m.forward(x, pre)
    for ladder, nm in () if not with_c1 else (((1, 3, 9), "c1"), ((1, 3, 9, 81), "c1b")):
        spec = synth.spec_c1(ladder)
        conf, w = synth.write_ncp(spec, tmp)
        out[f"sha_{nm}"] = np.frombuffer(bytes.fromhex(sha(w)), np.uint8)
        m = orc.Model(conf, w)
        pre = synth.ncp_prefixes(spec, 4, 7)
        out[f"codes_{nm}_greedy"] = m.generate(pre, temp=0.0)
        out[f"codes_{nm}_topk"] = m.generate(pre, temp=0.8, top_k=50, top_p=0.9, seed=3)


def orc_lms(out, tmp):
    import orc
    for kind, spec in (("gpt2", synth.spec_gpt2_tiny()), ("qwen", synth.spec_qwen_tiny())):
        conf, w = synth.write_lm(spec, tmp)
        out[f"sha_{kind}"] = np.frombuffer(bytes.fromhex(sha(w)), np.uint8)
        m = orc.LM(conf, w, kind == "qwen")
        prompts = synth.lm_prompts(spec, 2, 9, 3)
        for i, pr in enumerate(prompts):
            out[f"lm_{kind}_logits{i}"] = m.logits(pr)
            out[f"lm_{kind}_nll{i}"] = np.array([m.nll(pr)], np.float64)
            for tag, (t, tk, tp, sd) in (("greedy", (0.0, 0, 1.0, 0)), ("sampled", (0.7, 0, 0.95, 9)), ("topk", (0.9, 8, 1.0, 5))):
                out[f"lm_{kind}_gen{i}_{tag}"] = m.generate(pr, 12, temp=t, top_k=tk, top_p=tp, seed=sd)


def same_bits(a, b):
    """Bit equality that treats -inf == -inf and NaN == NaN by representation."""
    a, b = np.asarray(a), np.asarray(b)
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    return a.tobytes() == b.tobytes()


def top2_gap(row):
    top = np.partition(np.asarray(row, np.float64), -2)[-2:]
    return abs(top[1] - top[0]) / max(abs(top[1]), 1e-30)


def decoded_tokens_equal_or_near_tie(gm, om, codes, spec, tag):
    """token ids from the library's decoder against the oracle's on the same codes; a differing position is
    accepted only when the oracle's decoder logits there have a top-2 gap within 1e-5 relative"""
    tok_g = gm.decode_tokens(codes, spec.L)
    tok_o = om.decode_tokens(codes)
    diff = np.argwhere(tok_g != tok_o)
    ties = 0
    if len(diff):
        zh = om.idx_to_zhats(codes, len(spec.levels))
        lg = om.decode(zh[-1])
        for b, t in diff:
            gap = top2_gap(lg[b, t])
            assert gap <= 1e-5, f"{tag}: token ({b},{t}) differs, oracle top-2 gap {gap:.2e}"
            assert tok_g[b, t] in np.argsort(lg[b, t])[-2:]
            ties += 1
    print(f"{tag}: {tok_g.size} decoded tokens, {ties} near-ties")
    return tok_g
