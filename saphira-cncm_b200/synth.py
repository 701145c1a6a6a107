"""Seeded synthetic models and inputs for the token-loop configurations.

Writes the reference's on-disk formats so that the same files drive the CPU
oracle, the reference CPU build and the CUDA library:

* ``.ncm``  -- magic ``NCM1``, u32 tensor count, then per tensor: u8 name length,
  name, u8 ndim, u32 dims, u64 byte count, raw little-endian float32
  (layout read by the reference loader, src/tensor.c:70-128; same writer shape
  as tools/mkinit.py:118-132).
* ``.conf`` -- flat ``key=value`` lines (parsed by src/tensor.c:170-266).

Tensor names follow the lookups in src/ncp.c, src/vq.c, src/vqvae.c,
src/gpt2.c:54-75 and src/qwen.c:55-74.  Weights are N(0, 0.02); norm gains are 1
and biases 0 unless ``rand_affine`` is set (tests use it so that bias and gain
paths carry signal).  Inputs are drawn with ``numpy.random.default_rng(seed)``.

No public dataset is involved: every prefix, prompt and vector is synthetic.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass, field

import numpy as np


# --------------------------------------------------------------------------
# file writers
# --------------------------------------------------------------------------

def write_ncm(path: str, tensors: "dict[str, np.ndarray]") -> None:
    with open(path, "wb") as f:
        f.write(b"NCM1")
        f.write(struct.pack("<I", len(tensors)))
        for name, arr in tensors.items():
            t = np.ascontiguousarray(arr, dtype=np.float32)
            nb = name.encode()
            assert len(nb) < 256 and 1 <= t.ndim <= 4, name
            f.write(struct.pack("<B", len(nb)))
            f.write(nb)
            f.write(struct.pack("<B", t.ndim))
            for d in t.shape:
                f.write(struct.pack("<I", d))
            raw = t.tobytes()
            f.write(struct.pack("<Q", len(raw)))
            f.write(raw)


def write_ncm2(path: str, tensors: "dict[str, np.ndarray]", bf16: "bool | set[str]" = True) -> None:
    """The 2-byte variant of the weights file (magic ``NCM2``): the NCM1 layout with one byte of element type
    (0 = float32, 1 = bfloat16) in front of each record's byte count. Tensors with two or more dimensions (or the
    names in `bf16`) are written as bf16 bits -- their values must already be bf16 values -- the rest as float32."""
    with open(path, "wb") as f:
        f.write(b"NCM2")
        f.write(struct.pack("<I", len(tensors)))
        for name, arr in tensors.items():
            t = np.ascontiguousarray(arr, dtype=np.float32)
            half = (t.ndim >= 2) if isinstance(bf16, bool) and bf16 else (not isinstance(bf16, bool) and name in bf16)
            nb = name.encode()
            f.write(struct.pack("<B", len(nb)))
            f.write(nb)
            f.write(struct.pack("<B", t.ndim))
            for d in t.shape:
                f.write(struct.pack("<I", d))
            if half:
                bits = t.view(np.uint32)
                assert not (bits & 0xFFFF).any(), f"{name}: not a bf16 value"
                raw = (bits >> 16).astype(np.uint16).tobytes()
            else:
                raw = t.tobytes()
            f.write(struct.pack("<BQ", 1 if half else 0, len(raw)))
            f.write(raw)


def _fnv1a64(data: bytes) -> int:
    """FNV-1a 64 (a serial chain; fine for the small files tests write)."""
    h = 14695981039346656037
    mask = (1 << 64) - 1
    for b in data:
        h = ((h ^ b) * 1099511628211) & mask
    return h


def write_nck1(path: str, tensors: "dict[str, np.ndarray]", step: int = 7, optimizer_slots: int = 1) -> None:
    """A training checkpoint in the reference's NCK1 v1 layout (writer: src/ckpt.c:200-262): run-state header, the
    tensor records (same record layout as NCM1), an AdamW section, FNV-1a 64 of everything before it in the last
    eight bytes. Inference reads the tensor records only; the run state and the moments written here are filler of
    the right shape (moments for the first `optimizer_slots` tensors)."""
    out = bytearray()
    out += b"NCK1" + struct.pack("<I", 1)
    out += struct.pack("<qQdddiiqiQ", step, 0x9E3779B97F4A7C15, 3e-4, 100.0, 1000.0, 8, 0, 1234, 81, 0xABCDEF)
    for sfield in (b"data/train.bin",):
        out += struct.pack("<H", len(sfield)) + sfield
    out += struct.pack("<Q", 0x1234)
    for sfield in (b"sudoku", b'{"lr": 0.0003}'):
        out += struct.pack("<H", len(sfield)) + sfield
    out += struct.pack("<I", len(tensors))
    arrs = []
    for name, arr in tensors.items():
        t = np.ascontiguousarray(arr, dtype=np.float32)
        nb = name.encode()
        assert 0 < len(nb) < 256 and 1 <= t.ndim <= 4, name
        out += struct.pack("<B", len(nb)) + nb + struct.pack("<B", t.ndim)
        for d in t.shape:
            out += struct.pack("<I", d)
        raw = t.tobytes()
        out += struct.pack("<Q", len(raw)) + raw
        arrs.append(t)
    n_opt = min(optimizer_slots, len(arrs))
    out += b"ADAM" + struct.pack("<ddddIq", 0.9, 0.95, 1e-8, 0.1, n_opt, step)
    for i in range(n_opt):
        nbytes = arrs[i].size * 4
        out += struct.pack("<IdQ", i, 3e-4, nbytes) + bytes(nbytes) + struct.pack("<Q", nbytes) + bytes(nbytes)
    out += struct.pack("<Q", _fnv1a64(bytes(out)))
    with open(path, "wb") as f:
        f.write(out)


def _to_f16_bits(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float16).view(np.uint16)


def _to_bf16_bits(a: np.ndarray) -> np.ndarray:
    return (_round_bf16_early(a).view(np.uint32) >> 16).astype(np.uint16)


def _round_bf16_early(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def write_safetensors(path: str, tensors: "dict[str, np.ndarray]", dtypes: "dict[str, str] | str" = "F32",
                      metadata: "dict[str, str] | None" = None) -> None:
    """A Hugging Face .safetensors file: u64 header length, JSON header (name -> dtype, shape, data_offsets),
    then the tensors' bytes. dtypes: one of F32 / F16 / BF16 for all tensors, or per tensor name."""
    import json
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, arr in tensors.items():
        dt = dtypes if isinstance(dtypes, str) else dtypes.get(name, "F32")
        a = np.ascontiguousarray(arr, np.float32)
        raw = {"F32": lambda x: x.tobytes(), "F16": lambda x: _to_f16_bits(x).tobytes(),
               "BF16": lambda x: _to_bf16_bits(x).tobytes()}[dt](a)
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def lm_tensors_hf(s: "LMSpec", seed: int) -> "dict[str, np.ndarray]":
    """The tensors of lm_tensors() as a Hugging Face checkpoint stores them: GPT-2's Conv1D matrices [in][out]
    and a causal-mask buffer per layer; Qwen2's nn.Linear matrices unchanged."""
    out = {}
    for name, a in lm_tensors(s, seed).items():
        if s.kind == "gpt2" and a.ndim == 2 and name.endswith(".weight") and any(k in name for k in ("c_attn", "c_proj", "c_fc")):
            a = np.ascontiguousarray(a.T)
        out[name] = a
        if s.kind == "gpt2" and name.endswith("attn.c_attn.weight"):
            out[name[:-len("c_attn.weight")] + "bias"] = np.tril(np.ones((1, 1, 8, 8), np.float32))
    return out


def write_conf(path: str, kv: "dict[str, object]") -> None:
    with open(path, "w") as f:
        for k, v in kv.items():
            if isinstance(v, (list, tuple)):
                v = ",".join(str(x) for x in v)
            f.write(f"{k}={v}\n")


# --------------------------------------------------------------------------
# NCP + VQ-VAE
# --------------------------------------------------------------------------

@dataclass
class NCPSpec:
    name: str
    n_layer: int
    n_embd: int
    n_head: int
    n_kv_heads: int
    prefix_len: int
    levels: "list[int]"
    vocab: "list[int]"            # per quantizer level (also per head)
    vq_dim: int = 64
    in_vocab: int = 12
    vq_heads: int = 4             # vq.n_layers is the head count of the VAE blocks
    enc_layers: int = 2
    dec_layers: int = 2
    mlp_hidden: int = 0           # 0 -> 4*n_embd (ungated) / given (gated)
    swiglu: int = 0
    geglu: int = 0
    relu2: int = 0
    ln_bias: int = 1
    lin_bias: int = 1
    qk_norm: int = 0
    vq_qk_norm: int = 0
    use_rope: int = 1
    rope_base: int = 10000
    query_level0: int = 1
    pad_id: int = -1              # model.prefix_pad_token_id
    eos_id: int = -1
    tok_kind: str = "sudoku"
    l1_cascade: "list[int]" = field(default_factory=list)   # conv strides, product = levels[-1]/levels[0]
    l1_norm: int = 0
    l1_norm_final: int = 0
    qr_enabled: int = 0
    qr_ratio: float = 0.5
    qr_share: int = 0
    all_sampling: int = 0
    puc: int = 0
    puc_kernel: int = 3
    head_mode: str = "untied"     # untied | shared | shared_lvlbias | tied
    attn_block_diag: int = 1
    enc_positional: int = 0
    dec_positional: int = 0
    enc_convs: int = 0
    enc_conv_kernel: int = 3
    enc_window: int = 0
    pre_quant_gn: int = 0
    token_unigram: int = 0        # emit inference.token_unigram (uniform)
    rand_affine: int = 0
    gen: "dict[str, object]" = field(default_factory=dict)

    @property
    def L(self) -> int:
        return self.levels[-1]

    @property
    def total(self) -> int:
        return sum(self.levels)


def _mk(rng, shape, std=0.02):
    return rng.normal(0.0, std, size=shape).astype(np.float32)


def _gain(rng, n, rand):
    return (1.0 + rng.normal(0, 0.1, size=n)).astype(np.float32) if rand else np.ones(n, np.float32)


def _bias(rng, n, rand):
    return _mk(rng, (n,)) if rand else np.zeros(n, np.float32)


def _vae_block(t, rng, pre, D, heads, qk_norm, rand):
    t[pre + "ln_1.weight"] = _gain(rng, D, rand)
    t[pre + "ln_1.bias"] = _bias(rng, D, rand)
    t[pre + "attn.c_attn.weight"] = _mk(rng, (3 * D, D))
    t[pre + "attn.c_attn.bias"] = _bias(rng, 3 * D, rand)
    t[pre + "attn.c_proj.weight"] = _mk(rng, (D, D))
    t[pre + "attn.c_proj.bias"] = _bias(rng, D, rand)
    if qk_norm:
        t[pre + "attn.q_norm.weight"] = _gain(rng, D // heads, rand)
        t[pre + "attn.k_norm.weight"] = _gain(rng, D // heads, rand)
    t[pre + "ln_2.weight"] = _gain(rng, D, rand)
    t[pre + "ln_2.bias"] = _bias(rng, D, rand)
    t[pre + "mlp.c_fc.weight"] = _mk(rng, (4 * D, D))
    t[pre + "mlp.c_fc.bias"] = _bias(rng, 4 * D, rand)
    t[pre + "mlp.c_proj.weight"] = _mk(rng, (D, 4 * D))
    t[pre + "mlp.c_proj.bias"] = _bias(rng, D, rand)


def ncp_tensors(s: NCPSpec, seed: int) -> "dict[str, np.ndarray]":
    rng = np.random.default_rng(seed)
    t: "dict[str, np.ndarray]" = {}
    D, C, H = s.vq_dim, s.n_embd, s.n_head
    hd = C // H
    ra = s.rand_affine
    nl = len(s.levels)
    # --- tokenizer VQ-VAE ---
    t["tok.encoder.wte.weight"] = _mk(rng, (s.in_vocab, D))
    if s.enc_positional:
        t["tok.encoder.wpe.weight"] = _mk(rng, (s.L, D))
    for i in range(s.enc_convs):
        p = f"tok.encoder.conv_blocks.{i}."
        t[p + "ln.weight"] = _gain(rng, D, ra)
        t[p + "c1.weight"] = _mk(rng, (D, D, s.enc_conv_kernel))
        t[p + "c1.bias"] = _bias(rng, D, ra)
        t[p + "c2.weight"] = _mk(rng, (D, D, s.enc_conv_kernel))
        t[p + "c2.bias"] = _bias(rng, D, ra)
    for i in range(s.enc_layers):
        _vae_block(t, rng, f"tok.encoder.blocks.{i}.", D, s.vq_heads, s.vq_qk_norm, ra)
    t["tok.encoder.ln_e.weight"] = _gain(rng, D, ra)
    for i in range(nl):
        t[f"tok.vq.embeddings.{i}.weight"] = _mk(rng, (s.vocab[i], D))
    if s.qr_enabled:
        nphi = nl if s.qr_share == 0 else (1 if s.qr_share == 1 else s.qr_share)
        for i in range(nphi):
            t[f"tok.vq.quant_resi.{i}.weight"] = _mk(rng, (D, D, 3))
            t[f"tok.vq.quant_resi.{i}.bias"] = _bias(rng, D, ra)
    if s.l1_cascade:
        prod = 1
        for k in s.l1_cascade:
            prod *= k
        assert s.levels[0] * prod == s.L, "cascade strides must take levels[0] to L"
        # module indices skip the (weight-free) GroupNorm layers, like a torch Sequential
        idx = 0
        for j, k in enumerate(reversed(s.l1_cascade)):
            if s.l1_norm and j > 0:
                idx += 1
            t[f"tok.vq.learned_down_l1.{idx}.weight"] = _mk(rng, (D, D, k))
            t[f"tok.vq.learned_down_l1.{idx}.bias"] = _bias(rng, D, ra)
            idx += 1
        idx = 0
        for j, k in enumerate(s.l1_cascade):
            if s.l1_norm and j > 0:
                idx += 1
            t[f"tok.vq.learned_up_l1.{idx}.weight"] = _mk(rng, (D, D, k))
            t[f"tok.vq.learned_up_l1.{idx}.bias"] = _bias(rng, D, ra)
            idx += 1
    if s.all_sampling:
        for i in range(1, nl - 1):
            t[f"tok.vq.learned_down_refine.{i}.weight"] = _mk(rng, (D, D, 3))
            t[f"tok.vq.learned_down_refine.{i}.bias"] = _bias(rng, D, ra)
            t[f"tok.vq.learned_up_refine.{i}.weight"] = _mk(rng, (D, D, 3))
            t[f"tok.vq.learned_up_refine.{i}.bias"] = _bias(rng, D, ra)
    if s.dec_positional:
        t["tok.decoder.wpe.weight"] = _mk(rng, (s.L, D))
    _vae_block(t, rng, "tok.decoder.middle_block.", D, s.vq_heads, s.vq_qk_norm, ra)
    for i in range(s.dec_layers - 1):
        _vae_block(t, rng, f"tok.decoder.extra_blocks.{i}.", D, s.vq_heads, s.vq_qk_norm, ra)
    t["tok.decoder.ln_f.weight"] = _gain(rng, D, ra)
    t["tok.decoder.output_layer.weight"] = _mk(rng, (s.in_vocab, D))
    # --- NCP transformer ---
    lvl_first = 0 if s.query_level0 else 1
    n_tgt = nl - lvl_first
    t["gen.l0_queries"] = _mk(rng, (1, s.levels[0], D))
    t["gen.transformer.wte.weight"] = _mk(rng, (C, D))
    t["gen.transformer.wte.bias"] = _bias(rng, C, ra)
    t["gen.transformer.wle.weight"] = _mk(rng, (max(n_tgt, 1), C))
    if not s.use_rope:
        t["gen.transformer.wpe.weight"] = _mk(rng, (max(s.prefix_len, max(s.levels)), C))
    gated = s.swiglu or s.geglu
    Hh = s.mlp_hidden if s.mlp_hidden else 4 * C
    nqkv = C + 2 * s.n_kv_heads * hd
    for b in range(s.n_layer):
        p = f"gen.transformer.blocks.{b}."
        t[p + "ln_1.weight"] = _gain(rng, C, ra)
        if s.ln_bias:
            t[p + "ln_1.bias"] = _bias(rng, C, ra)
        t[p + "attn.c_attn.weight"] = _mk(rng, (nqkv, C))
        if s.lin_bias:
            t[p + "attn.c_attn.bias"] = _bias(rng, nqkv, ra)
        t[p + "attn.c_proj.weight"] = _mk(rng, (C, C))
        if s.lin_bias:
            t[p + "attn.c_proj.bias"] = _bias(rng, C, ra)
        if s.qk_norm:
            t[p + "attn.q_norm.weight"] = _gain(rng, hd, ra)
            t[p + "attn.k_norm.weight"] = _gain(rng, hd, ra)
        t[p + "ln_2.weight"] = _gain(rng, C, ra)
        if s.ln_bias:
            t[p + "ln_2.bias"] = _bias(rng, C, ra)
        if gated:
            t[p + "mlp.w_gate.weight"] = _mk(rng, (Hh, C))
            t[p + "mlp.w_up.weight"] = _mk(rng, (Hh, C))
            if s.lin_bias:
                t[p + "mlp.w_gate.bias"] = _bias(rng, Hh, ra)
                t[p + "mlp.w_up.bias"] = _bias(rng, Hh, ra)
        else:
            t[p + "mlp.c_fc.weight"] = _mk(rng, (Hh, C))
            if s.lin_bias:
                t[p + "mlp.c_fc.bias"] = _bias(rng, Hh, ra)
        t[p + "mlp.c_proj.weight"] = _mk(rng, (C, Hh))
        if s.lin_bias:
            t[p + "mlp.c_proj.bias"] = _bias(rng, C, ra)
    t["gen.transformer.ln_f.weight"] = _gain(rng, C, ra)
    if s.ln_bias:
        t["gen.transformer.ln_f.bias"] = _bias(rng, C, ra)
    head_vocab = s.vocab[lvl_first:]
    if s.head_mode in ("shared", "shared_lvlbias"):
        t["gen.lm_heads.head.weight"] = _mk(rng, (head_vocab[0], C))
        if s.head_mode == "shared_lvlbias":
            for k in range(n_tgt):
                t[f"gen.lm_heads.biases.{k}"] = _mk(rng, (head_vocab[k],))
    elif s.head_mode == "tied":
        for k in range(n_tgt):
            t[f"gen.lm_heads.{k}.proj.weight"] = _mk(rng, (D, C))
            t[f"gen.lm_heads.{k}.proj.bias"] = _bias(rng, D, ra)
            t[f"gen.lm_heads.{k}.log_inv_T"] = np.array([0.3], np.float32)
            t[f"gen.lm_heads.{k}.bias"] = _mk(rng, (head_vocab[k],))
    else:
        for k in range(n_tgt):
            t[f"gen.lm_heads.{k}.weight"] = _mk(rng, (head_vocab[k], C))
            t[f"gen.lm_heads.{k}.bias"] = _bias(rng, head_vocab[k], ra)
    if s.puc:
        for k in range(n_tgt):
            t[f"gen.post_upsample_convs.{k}.weight"] = _mk(rng, (D, D, s.puc_kernel))
            t[f"gen.post_upsample_convs.{k}.bias"] = _bias(rng, D, ra)
    if s.token_unigram:
        vmax = max(head_vocab)
        t["inference.token_unigram"] = np.full((vmax,), 1.0 / vmax, np.float32)
    return t


def ncp_conf(s: NCPSpec) -> "dict[str, object]":
    lvl_first = 0 if s.query_level0 else 1
    kv: "dict[str, object]" = {
        "task": s.name,
        "model.n_layer": s.n_layer, "model.n_head": s.n_head, "model.n_embd": s.n_embd,
        "model.n_kv_heads": s.n_kv_heads,
        "model.prefix_len": s.prefix_len, "model.bias": s.lin_bias,
        "model.raw_token_prefix": 1, "model.prefix_pad_token_id": s.pad_id,
        "model.query_level0": s.query_level0,
        "model.attn_pattern": "block_diagonal" if s.attn_block_diag else "block_causal",
        "model.use_rope": s.use_rope, "model.rope_base": s.rope_base,
        "model.use_qk_norm": s.qk_norm,
        "model.use_swiglu": s.swiglu, "model.use_geglu": s.geglu, "model.use_relu2": s.relu2,
        "model.puc_enabled": s.puc, "model.puc_kernel": s.puc_kernel,
        "model.shared_output_head": 1 if s.head_mode.startswith("shared") else 0,
        "model.shared_head_per_level_bias": 1 if s.head_mode == "shared_lvlbias" else 0,
        "model.tie_heads_to_codebook": 1 if s.head_mode == "tied" else 0,
        "model.vocab_size": s.vocab[lvl_first:],
        "vq.embed_dim": s.vq_dim, "vq.in_vocab": s.in_vocab,
        "vq.context_length": s.L, "vq.n_layers": s.vq_heads, "vq.compression": 1,
        "vq.levels": s.levels, "vq.vocab": s.vocab,
        "vq.qr_enabled": s.qr_enabled, "vq.qr_ratio": s.qr_ratio, "vq.qr_share": s.qr_share,
        "vq.l1_sampling": 1 if s.l1_cascade else 0, "vq.l1_cascade": 1 if s.l1_cascade else 0,
        "vq.l1_norm": s.l1_norm, "vq.l1_norm_final": s.l1_norm_final,
        "vq.all_sampling": s.all_sampling, "vq.pre_quant_gn": s.pre_quant_gn,
        "vq.qk_norm": s.vq_qk_norm,
        "vq.enc_layers": s.enc_layers, "vq.enc_window": s.enc_window,
        "vq.enc_convs": s.enc_convs, "vq.enc_conv_kernel": s.enc_conv_kernel,
        "vq.enc_positional": s.enc_positional,
        "vq.dec_layers": s.dec_layers, "vq.dec_positional": s.dec_positional,
        "tok.kind": s.tok_kind, "tok.eos_id": s.eos_id, "tok.pad_id": s.pad_id,
    }
    for k, v in s.gen.items():
        kv["gen." + k] = v
    return kv


def zipf_ids(rng, n, lo, hi, a=1.1):
    """Zipf(a)-distributed ids on [lo, hi) (rank r has weight r**-a)."""
    ranks = np.arange(1, hi - lo + 1, dtype=np.float64)
    p = ranks ** (-a)
    p /= p.sum()
    return (lo + rng.choice(hi - lo, size=n, p=p)).astype(np.int32)


def ncp_prefixes(s: NCPSpec, B: int, seed: int) -> np.ndarray:
    """[B, prefix_len] int32 prefixes with the distribution the configuration states."""
    rng = np.random.default_rng(seed ^ 0x5EED)
    P = s.prefix_len
    if s.tok_kind == "sudoku":
        cells = rng.integers(1, 10, size=(B, P))
        keep = rng.random((B, P)) >= 0.5
        return np.where(keep, cells, 0).astype(np.int32)
    lo = 2 if (s.pad_id >= 0 or s.eos_id >= 0) else 0      # never pad / eos
    return zipf_ids(rng, B * P, lo, s.in_vocab).reshape(B, P)


# named configurations -------------------------------------------------------

def spec_c1(ladder=(1, 3, 9)) -> NCPSpec:
    """Small NCP + VQ-VAE (4 x 256 x 8 heads, codebook 512 x 64, greedy)."""
    lv = list(ladder)
    return NCPSpec(name="c1" if len(lv) == 3 else "c1b", n_layer=4, n_embd=256, n_head=8,
                   n_kv_heads=8, prefix_len=81, levels=lv, vocab=[512] * len(lv),
                   vq_dim=64, in_vocab=12, vq_heads=4, enc_layers=2, dec_layers=2,
                   tok_kind="sudoku", gen={"temperature": 0.0})


def spec_c2(n_layer=12, n_embd=512, n_head=8, n_kv=2, vocab=4096, name="c2") -> NCPSpec:
    """Mid NCP with GQA, SwiGLU 4x, CFG, learned L1 cascade with GroupNorm(8)."""
    return NCPSpec(name=name, n_layer=n_layer, n_embd=n_embd, n_head=n_head, n_kv_heads=n_kv,
                   prefix_len=256, levels=[1, 4, 16, 32], vocab=[vocab] * 4,
                   vq_dim=64, in_vocab=8192, vq_heads=4, enc_layers=2, dec_layers=2,
                   mlp_hidden=4 * n_embd, swiglu=1, ln_bias=0, lin_bias=1,
                   pad_id=0, eos_id=1, tok_kind="bpe",
                   l1_cascade=[2, 4, 4], l1_norm=1, token_unigram=1,
                   gen={"temperature": 0.8, "top_k": 50, "top_p": 0.9,
                        "cfg_scale": 1.5, "freq": 0.2})


def spec_c5() -> NCPSpec:
    """Box-scale NCP: config-2 shape at 24 x 1024 x 16/4 heads, codebook 16384 x 64."""
    return spec_c2(n_layer=24, n_embd=1024, n_head=16, n_kv=4, vocab=16384, name="c5")


def spec_tiny(**over) -> NCPSpec:
    """A seconds-scale model that switches on every optional path at once."""
    base = dict(name="tiny", n_layer=2, n_embd=64, n_head=4, n_kv_heads=2, prefix_len=12,
                levels=[1, 2, 4, 8], vocab=[32, 32, 32, 32], vq_dim=32, in_vocab=24,
                vq_heads=4, enc_layers=1, dec_layers=2, mlp_hidden=96, swiglu=1,
                ln_bias=1, lin_bias=1, qk_norm=1, vq_qk_norm=1, pad_id=0, eos_id=1,
                tok_kind="bpe", l1_cascade=[2, 4], l1_norm=1, l1_norm_final=1,
                qr_enabled=1, qr_ratio=0.5, qr_share=0, all_sampling=1, puc=1,
                token_unigram=1, rand_affine=1, dec_positional=1, enc_positional=1,
                gen={"temperature": 0.8, "top_k": 5, "top_p": 0.9, "cfg_scale": 1.5,
                     "freq": 0.2, "mu": 0.1, "adj": "0.3,2,0.5"})
    base.update(over)
    return NCPSpec(**base)


def write_ncp(s: NCPSpec, out_dir: str, seed: int = 1234) -> "tuple[str, str]":
    os.makedirs(out_dir, exist_ok=True)
    w = os.path.join(out_dir, f"{s.name}.ncm")
    c = os.path.join(out_dir, f"{s.name}.conf")
    write_ncm(w, ncp_tensors(s, seed))
    write_conf(c, ncp_conf(s))
    return c, w


# --------------------------------------------------------------------------
# GPT-2 / Qwen2 shaped decoders
# --------------------------------------------------------------------------

@dataclass
class LMSpec:
    name: str
    kind: str              # gpt2 | qwen
    n_layer: int
    n_embd: int
    n_head: int
    n_kv_heads: int
    n_inner: int
    vocab: int
    n_ctx: int
    rope_theta: float = 1e6
    bf16_round: int = 0    # round weights to bf16 (stored as float32)
    rand_affine: int = 0


def _round_bf16(a: np.ndarray) -> np.ndarray:
    """round-to-nearest-even to bf16, kept as float32 (finite weights: the 32-bit add cannot wrap)"""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).copy()
    u += np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    u &= np.uint32(0xFFFF0000)
    return u.view(np.float32)


def lm_tensors(s: LMSpec, seed: int) -> "dict[str, np.ndarray]":
    rng = np.random.default_rng(seed)
    C, ra = s.n_embd, s.rand_affine
    hd = C // s.n_head
    t: "dict[str, np.ndarray]" = {}
    if s.kind == "gpt2":
        t["wte.weight"] = _mk(rng, (s.vocab, C))
        t["wpe.weight"] = _mk(rng, (s.n_ctx, C))
        for i in range(s.n_layer):
            p = f"h.{i}."
            t[p + "ln_1.weight"] = _gain(rng, C, ra); t[p + "ln_1.bias"] = _bias(rng, C, ra)
            t[p + "attn.c_attn.weight"] = _mk(rng, (3 * C, C))
            t[p + "attn.c_attn.bias"] = _bias(rng, 3 * C, ra)
            t[p + "attn.c_proj.weight"] = _mk(rng, (C, C))
            t[p + "attn.c_proj.bias"] = _bias(rng, C, ra)
            t[p + "ln_2.weight"] = _gain(rng, C, ra); t[p + "ln_2.bias"] = _bias(rng, C, ra)
            t[p + "mlp.c_fc.weight"] = _mk(rng, (4 * C, C))
            t[p + "mlp.c_fc.bias"] = _bias(rng, 4 * C, ra)
            t[p + "mlp.c_proj.weight"] = _mk(rng, (C, 4 * C))
            t[p + "mlp.c_proj.bias"] = _bias(rng, C, ra)
        t["ln_f.weight"] = _gain(rng, C, ra); t["ln_f.bias"] = _bias(rng, C, ra)
    else:
        kvd = s.n_kv_heads * hd
        t["model.embed_tokens.weight"] = _mk(rng, (s.vocab, C))
        for i in range(s.n_layer):
            p = f"model.layers.{i}."
            t[p + "input_layernorm.weight"] = _gain(rng, C, ra)
            t[p + "self_attn.q_proj.weight"] = _mk(rng, (C, C))
            t[p + "self_attn.q_proj.bias"] = _bias(rng, C, ra)
            t[p + "self_attn.k_proj.weight"] = _mk(rng, (kvd, C))
            t[p + "self_attn.k_proj.bias"] = _bias(rng, kvd, ra)
            t[p + "self_attn.v_proj.weight"] = _mk(rng, (kvd, C))
            t[p + "self_attn.v_proj.bias"] = _bias(rng, kvd, ra)
            t[p + "self_attn.o_proj.weight"] = _mk(rng, (C, C))
            t[p + "post_attention_layernorm.weight"] = _gain(rng, C, ra)
            t[p + "mlp.gate_proj.weight"] = _mk(rng, (s.n_inner, C))
            t[p + "mlp.up_proj.weight"] = _mk(rng, (s.n_inner, C))
            t[p + "mlp.down_proj.weight"] = _mk(rng, (C, s.n_inner))
        t["model.norm.weight"] = _gain(rng, C, ra)
    if s.bf16_round:
        t = {k: _round_bf16(v) for k, v in t.items()}
    return t


def lm_conf(s: LMSpec) -> "dict[str, object]":
    kv = {"task": "gpt2" if s.kind == "gpt2" else "qwen2",
          "model.n_layer": s.n_layer, "model.n_head": s.n_head, "model.n_embd": s.n_embd,
          "model.n_kv_heads": s.n_kv_heads, "model.context_length": s.n_ctx,
          "model.vocab_size": s.vocab, "model.bias": 1 if s.kind == "gpt2" else 0,
          "model.use_rope": 0, "model.use_qk_norm": 0, "model.prefix_pad_token_id": -1,
          "tok.kind": "sudoku",      # no tokenizer assets: ids in, ids out
          "tok.eos_id": -1, "tok.pad_id": -1}
    if s.kind == "qwen":
        kv["model.rope_theta"] = repr(float(s.rope_theta))
    return kv


def spec_gpt2_124m() -> LMSpec:
    return LMSpec("gpt2_124m", "gpt2", 12, 768, 12, 12, 3072, 50257, 1024)


def spec_gpt2_tiny() -> LMSpec:
    return LMSpec("gpt2_tiny", "gpt2", 2, 64, 4, 4, 256, 211, 64, rand_affine=1)


def spec_qwen_05b() -> LMSpec:
    return LMSpec("qwen_05b", "qwen", 24, 896, 14, 2, 4864, 151936, 1024, rope_theta=1e6,
                  bf16_round=1)


def spec_qwen_tiny() -> LMSpec:
    return LMSpec("qwen_tiny", "qwen", 2, 64, 4, 2, 160, 307, 64, rope_theta=1e6,
                  rand_affine=1)


def write_lm(s: LMSpec, out_dir: str, seed: int = 4321) -> "tuple[str, str]":
    os.makedirs(out_dir, exist_ok=True)
    w = os.path.join(out_dir, f"{s.name}.ncm")
    c = os.path.join(out_dir, f"{s.name}.conf")
    write_ncm(w, lm_tensors(s, seed))
    write_conf(c, lm_conf(s))
    return c, w


def lm_prompts(s: LMSpec, B: int, n: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed ^ 0xABCD)
    return zipf_ids(rng, B * n, 0, s.vocab).reshape(B, n)
