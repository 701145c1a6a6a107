"""Case list shared by the golden-vector generator and the tests that read them.

Every case is small enough for the CPU reference to finish in well under a
second; inputs are regenerated from seeds, outputs are stored in golden.npz.
"""
import numpy as np

import synth

# sampling settings exercised on the tiny NCP model
SAMPLERS = {
    "greedy": dict(temp=0.0),
    "topk": dict(temp=0.8, top_k=5, top_p=0.9, seed=5),
    "cfg": dict(temp=0.8, top_k=5, top_p=0.9, cfg=1.5, seed=7),
    "cfg_pen": dict(temp=0.8, top_k=5, top_p=0.9, cfg=1.5, freq=0.2, mu=0.1, adj=(0.3, 2, 0.5),
                    seed=11, allow=True),
    "nucleus": dict(temp=1.0, top_k=0, top_p=0.7, seed=13),
    # penalties that only lower logits (no deficit bonus): the case the two-phase device sampler covers
    "cfg_pen_down": dict(temp=0.8, top_k=5, top_p=0.9, cfg=1.5, freq=0.2, adj=(0.3, 2, 0.5), seed=17, allow=True),
}

# tiny NCP variants: name -> spec overrides
NCP_VARIANTS = {
    "full": dict(),
    "tied": dict(head_mode="tied", vocab=[48, 40, 32, 32],
                 gen={}),                       # no adjacency with unequal vocabularies
    "shared": dict(head_mode="shared_lvlbias", swiglu=0, geglu=1),
    "norope_relu2": dict(use_rope=0, swiglu=0, relu2=1, mlp_hidden=0, qr_share=1),
    "plain": dict(qk_norm=0, vq_qk_norm=0, l1_cascade=[], l1_norm=0, l1_norm_final=0,
                  qr_enabled=0, all_sampling=0, puc=0, pad_id=-1, eos_id=-1, swiglu=0,
                  mlp_hidden=0, n_kv_heads=4, enc_convs=1, enc_window=2, pre_quant_gn=4),
    "given_l0": dict(query_level0=0),
    "causal": dict(attn_block_diag=0),           # block-causal level pattern in the teacher-forced forward
}


def ncp_spec(variant: str) -> "synth.NCPSpec":
    over = dict(NCP_VARIANTS[variant])
    over.setdefault("name", "tiny_" + variant)
    return synth.spec_tiny(**over)


def ncp_inputs(spec, B=3, seed=7):
    pre = synth.ncp_prefixes(spec, B, seed)
    if spec.pad_id >= 0:
        pre[0, -3:] = spec.pad_id            # one row with trailing pads
        pre[B - 1, 2] = spec.pad_id          # and one with an interior pad
    rng = np.random.default_rng(seed + 1)
    l0 = rng.integers(0, spec.vocab[0], size=(B, spec.levels[0])).astype(np.int32)
    ids = rng.integers(0, spec.in_vocab, size=(B, spec.L)).astype(np.int32)
    return pre, l0, ids


def sampler_kwargs(name: str, spec):
    kw = dict(SAMPLERS[name])
    if kw.pop("allow", False):
        kw["allow"] = np.full(max(spec.vocab), 1.0 / max(spec.vocab))
    if max(spec.vocab) != min(spec.vocab):
        kw.pop("adj", None)                  # reference indexes out of bounds otherwise
    return kw


def kernel_inputs():
    """Seeded inputs of the layer-kernel cases (shapes echo the reference's own
    kernel checksum harness, tests/ktest_kernels.c, plus GQA and odd sizes)."""
    r = np.random.default_rng(20241)
    f = lambda *s: r.uniform(-2, 2, size=s).astype(np.float32)
    d = {}
    d["lin_x"], d["lin_W"], d["lin_b"] = f(8, 64), f(128, 64), f(128)
    d["lin2_x"], d["lin2_W"] = f(5, 37), f(19, 37)
    d["ln_x"], d["ln_w"], d["ln_b"] = f(4, 64), f(64), f(64)
    d["act_x"] = f(512)
    d["rope_q"], d["rope_k"] = f(1, 2, 16, 32), f(1, 2, 16, 32)
    d["rope_cos"], d["rope_sin"] = f(16, 32), f(16, 32)
    d["sd_q"], d["sd_k"], d["sd_v"] = f(1, 2, 8, 16), f(1, 2, 12, 16), f(1, 2, 12, 16)
    m = f(8, 12)
    d["sd_mask"] = np.where(m > 0, 0.0, -np.inf).astype(np.float32)
    d["sd_mask"][:, 0] = 0.0                 # no fully masked row
    d["gq_q"], d["gq_k"], d["gq_v"] = f(2, 4, 5, 8), f(2, 2, 7, 8), f(2, 2, 7, 8)
    d["cv_x"], d["cv_W"], d["cv_b"] = f(2, 4, 32), f(4, 4, 3), f(4)
    d["cs_W"] = f(4, 4, 2)                   # strided conv / conv-transpose, K = stride
    d["ar_x"] = f(2, 4, 32)
    d["li_x"] = f(2, 4, 9)
    d["l2_a"], d["l2_b"] = f(16, 32), f(8, 32)
    d["smp"] = f(6, 50)
    # data-movement / element-wise kernels (drawn after everything above, so the earlier inputs keep their values)
    d["emb_W"] = f(37, 24)
    d["emb_idx"] = r.integers(0, 37, size=19).astype(np.int32)
    d["rg_q"], d["rg_k"] = f(2, 6, 5, 16), f(2, 2, 5, 16)          # 6 query heads on 2 kv heads
    d["rg_cos"], d["rg_sin"] = f(5, 16), f(5, 16)
    d["ht_x"] = f(7, 3 * 8)                                        # [T][H*hd]
    d["htb_x"] = f(2, 7, 3 * 8)                                    # [B][T][H*hd]
    d["ew_a"], d["ew_b"] = f(1000), f(1000)
    d["qs_x"] = f(2, 5, 32 + 2 * 2 * 8)                            # [B][T][C + 2*K*hd], shapes in QS below
    d["hm_x"] = f(2, 3, 5, 8)
    return d


# qkv_split_fwd / head_merge_fwd shapes: B, T, C, H, hd, kv heads, query heads per kv head
QS = dict(B=2, T=5, C=32, H=4, hd=8, K=2, rep=2)
HM = dict(B=2, T=5, C=24, H=3, hd=8)
