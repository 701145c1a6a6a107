"""numpy-facing ctypes wrapper of the CPU oracle (oracle/liboracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and
by the CPU-baseline legs of ``bench.py``; never by the shipped package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libcncm_ref.so")

_P, _I, _F, _U64, _I64 = C.c_void_p, C.c_int, C.c_float, C.c_uint64, C.c_int64


def build(force: bool = False) -> str:
    """Compile liboracle.so (gcc, a few seconds) if it is missing or stale."""
    src = os.path.join(HERE, "oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
    return LIB


def reference_dir() -> "str | None":
    """Where the reference's source tree lies: $NCM_REFERENCE_DIR, else a directory named `reference` beside this
    repository. None when neither holds a src/ folder (the prebuilt oracle/_ref is used as it is then)."""
    cands = [os.environ.get("NCM_REFERENCE_DIR"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "src")):
            return c
    return None


def build_ref(ref_dir: "str | None" = None) -> "str | None":
    """Compile the reference CPU build into oracle/_ref/ when its sources exist."""
    ref_dir = ref_dir or reference_dir()
    if not ref_dir or not os.path.isdir(os.path.join(ref_dir, "src")):
        return REF_LIB if os.path.exists(REF_LIB) else None
    subprocess.check_call(["make", "-s", "-C", HERE, "ref", f"REF={ref_dir}"])
    # the reference's command-line front end linked against the GPU library (needs that library built)
    if os.path.exists(os.path.join(HERE, "..", "saphira-cncm_b200", "libncm_b200.so")):
        subprocess.check_call(["make", "-s", "-C", HERE, "cli", "ktest", f"REF={ref_dir}"])
    return REF_LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB, mode=os.RTLD_LOCAL | os.RTLD_NOW)
        sig = {
            "orc_linear": (None, [_P, _P, _P, _P, _I64, _I, _I]),
            "orc_layernorm": (None, [_P, _P, _P, _P, _I64, _I, C.c_double]),
            "orc_rmsnorm": (None, [_P, _P, _P, _I64, _I]),
            "orc_gelu": (None, [_P, _P, _I64]),
            "orc_gelu_tanh": (None, [_P, _P, _I64]),
            "orc_silu": (None, [_P, _P, _I64]),
            "orc_softmax": (None, [_P, _P, _I64, _I]),
            "orc_rope": (None, [_P, _P, _P, _I64, _I, _I]),
            "orc_sdpa": (None, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I]),
            "orc_conv1d": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I]),
            "orc_convT1d": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I]),
            "orc_groupnorm": (None, [_P, _P, _I, _I, _I, _I]),
            "orc_interp_area": (None, [_P, _P, _I, _I, _I, _I]),
            "orc_interp_linear": (None, [_P, _P, _I, _I, _I, _I]),
            "orc_l2sq": (None, [_P, _P, _P, _I64, _I64, _I]),
            "orc_argmax": (_I, [_P, _I]),
            "orc_rng_next": (_U64, [C.POINTER(_U64)]),
            "orc_sample_topkp": (_I, [_P, _I, _F, _I, _F, C.POINTER(_U64)]),
            "orc_model_load": (_P, [C.c_char_p, C.c_char_p]),
            "orc_model_free": (None, [_P]),
            "orc_total_codes": (_I, [_P]),
            "orc_L": (_I, [_P]),
            "orc_D": (_I, [_P]),
            "orc_in_vocab": (_I, [_P]),
            "orc_vq_z_to_idx": (None, [_P, _P, _I, _P]),
            "orc_vq_idx_to_zhats": (None, [_P, _P, _I, _P]),
            "orc_vq_next_input": (None, [_P, _P, _I, _P, _P, _I]),
            "orc_vq_idx_to_ncm_input": (None, [_P, _P, _I, _P]),
            "orc_vqvae_encode": (None, [_P, _P, _P, _I]),
            "orc_vqvae_decode": (None, [_P, _P, _P, _I]),
            "orc_decode_tokens": (None, [_P, _P, _I, _P]),
            "orc_ncp_generate": (None, [_P, _P, _P, _I, _F, _I, _F, _F, _F, _F, _F, _I, _F, _P,
                                        _U64, _P, _P]),
            "orc_ncp_forward": (None, [_P, _P, _P, _P, _I]),
            "orc_ncp_T": (_I, [_P]),
            "orc_ncp_maxV": (_I, [_P]),
            "orc_lm_load": (_P, [C.c_char_p, C.c_char_p, _I]),
            "orc_lm_free": (None, [_P]),
            "orc_lm_vocab": (_I, [_P]),
            "orc_lm_logits": (None, [_P, _P, _I, _I, _P]),
            "orc_lm_nll": (C.c_double, [_P, _P, _I]),
            "orc_lm_generate": (_I, [_P, _P, _I, _I, _F, _I, _F, _U64, _I, _P]),
        }
        for k, (r, a) in sig.items():
            fn = getattr(L, k)
            fn.restype, fn.argtypes = r, a
        _lib = L
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a):
    return None if a is None else a.ctypes.data


# ---- kernels --------------------------------------------------------------

def linear(x, W, b=None):
    x, W = _f(x), _f(W)
    b = None if b is None else _f(b)
    M, K = W.shape
    y = np.empty(x.shape[:-1] + (M,), np.float32)
    lib().orc_linear(_p(x), _p(W), _p(b), _p(y), x.size // K, M, K)
    return y


def layernorm(x, w=None, b=None, eps=1e-6):
    x = _f(x)
    w = None if w is None else _f(w)
    b = None if b is None else _f(b)
    y = np.empty_like(x)
    lib().orc_layernorm(_p(x), _p(w), _p(b), _p(y), x.size // x.shape[-1], x.shape[-1], eps)
    return y


def rmsnorm(x, w=None):
    x = _f(x)
    w = None if w is None else _f(w)
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), _p(y), x.size // x.shape[-1], x.shape[-1])
    return y


def _unary(name, x):
    x = _f(x)
    y = np.empty_like(x)
    getattr(lib(), name)(_p(x), _p(y), x.size)
    return y


def gelu(x):
    return _unary("orc_gelu", x)


def gelu_tanh(x):
    return _unary("orc_gelu_tanh", x)


def silu(x):
    return _unary("orc_silu", x)


def softmax(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().orc_softmax(_p(x), _p(y), x.size // x.shape[-1], x.shape[-1])
    return y


def rope(x, cs, sn, T):
    """x: [..., hd] with rows cycling through T table rows; returns rotated copy."""
    x = _f(x).copy()
    cs, sn = _f(cs), _f(sn)
    hd = x.shape[-1]
    lib().orc_rope(_p(x), _p(cs), _p(sn), x.size // hd, T, hd)
    return x


def sdpa(q, k, v, mask=None):
    """q: [B,Hq,Tq,hd], k/v: [B,Hkv,Tkv,hd], mask: [Tq,Tkv] additive or None."""
    q, k, v = _f(q), _f(k), _f(v)
    mask = None if mask is None else _f(mask)
    B, Hq, Tq, hd = q.shape
    Hkv, Tkv = k.shape[1], k.shape[2]
    out = np.empty_like(q)
    lib().orc_sdpa(_p(q), _p(k), _p(v), _p(mask), _p(out), B, Hq, Hkv, Tq, Tkv, hd)
    return out


def conv1d(x, W, b, stride, pad):
    x, W = _f(x), _f(W)
    b = None if b is None else _f(b)
    N, Cin, T = x.shape
    Cout, _, K = W.shape
    Tout = (T + 2 * pad - K) // stride + 1
    y = np.empty((N, Cout, Tout), np.float32)
    lib().orc_conv1d(_p(x), _p(W), _p(b), _p(y), N, Cin, Cout, T, K, stride, pad)
    return y


def convT1d(x, W, b, stride):
    x, W = _f(x), _f(W)
    b = None if b is None else _f(b)
    N, Cin, T = x.shape
    _, Cout, K = W.shape
    y = np.empty((N, Cout, (T - 1) * stride + K), np.float32)
    lib().orc_convT1d(_p(x), _p(W), _p(b), _p(y), N, Cin, Cout, T, K, stride)
    return y


def groupnorm(x, G):
    x = _f(x)
    N, Cc, T = x.shape
    y = np.empty_like(x)
    lib().orc_groupnorm(_p(x), _p(y), N, G, Cc, T)
    return y


def interp_area(x, Tout):
    x = _f(x)
    N, Cc, T = x.shape
    y = np.empty((N, Cc, Tout), np.float32)
    lib().orc_interp_area(_p(x), _p(y), N, Cc, T, Tout)
    return y


def interp_linear(x, Tout):
    x = _f(x)
    N, Cc, T = x.shape
    y = np.empty((N, Cc, Tout), np.float32)
    lib().orc_interp_linear(_p(x), _p(y), N, Cc, T, Tout)
    return y


def l2sq(a, b):
    a, b = _f(a), _f(b)
    d = np.empty((a.shape[0], b.shape[0]), np.float32)
    lib().orc_l2sq(_p(a), _p(b), _p(d), a.shape[0], b.shape[0], a.shape[1])
    return d


# Data-movement and element-wise kernels of the public kernel API: index arithmetic restated in numpy
# (fp32 throughout, one rounding per element like the reference's scalar loops).

def embedding(W, idx):
    """y[i, :] = W[idx[i], :]  (reference src/kernels.c:67-74)"""
    return _f(W)[_i(idx)].copy()


def rope_gqa(q, k, cs, sn):
    """q [B,H,T,hd], k [B,K,T,hd] rotated with the same [T,hd] tables, row r of either using table row r % T
    (reference src/kernels.c:299-309 on rope_one_exact, :270-283)."""
    T, hd = _f(cs).shape
    return rope(q, cs, sn, T), rope(k, cs, sn, T)


def heads_transpose(x, T, H, hd):
    """[T][H*hd] -> [H][T][hd]  (reference src/kernels.c:322-332)"""
    return np.ascontiguousarray(_f(x).reshape(T, H, hd).transpose(1, 0, 2))


def heads_transpose_b(x, B, T, H, hd):
    """[B][T][H*hd] -> [B][H][T][hd]  (reference src/kernels.c:345-357)"""
    return np.ascontiguousarray(_f(x).reshape(B, T, H, hd).transpose(0, 2, 1, 3))


def add(a, b):
    """reference src/kernels.c:843-849"""
    return _f(a) + _f(b)


def mul(a, b):
    """reference src/kernels.c:859-866"""
    return _f(a) * _f(b)


def scale(x, s):
    """y = x * s with s a float32 (reference src/kernels.c:868-874)"""
    return _f(x) * np.float32(s)


def qkv_split(x, B, T, C_, H, hd, K, rep):
    """[B,T,C+2*K*hd] -> q, k, v [B,H,T,hd]; query head h reads kv head h // rep (reference src/kernels.c:913-926)"""
    x = _f(x).reshape(B, T, C_ + 2 * K * hd)
    q = x[:, :, :H * hd].reshape(B, T, H, hd).transpose(0, 2, 1, 3)
    kk = x[:, :, C_:C_ + K * hd].reshape(B, T, K, hd).transpose(0, 2, 1, 3)
    vv = x[:, :, C_ + K * hd:].reshape(B, T, K, hd).transpose(0, 2, 1, 3)
    sel = np.arange(H) // rep
    return np.ascontiguousarray(q), np.ascontiguousarray(kk[:, sel]), np.ascontiguousarray(vv[:, sel])


def head_merge(ctx, B, T, C_, H, hd):
    """[B,H,T,hd] -> [B,T,C]  (reference src/kernels.c:928-936)"""
    return np.ascontiguousarray(_f(ctx).reshape(B, H, T, hd).transpose(0, 2, 1, 3).reshape(B, T, C_))


def sample_topkp(logits, temp, top_k, top_p, rng_state: int):
    """Returns (pick, new_rng_state)."""
    logits = _f(logits)
    st = _U64(rng_state)
    pick = lib().orc_sample_topkp(_p(logits), logits.size, temp, top_k, top_p, C.byref(st))
    return pick, st.value


def rng_stream(seed: int, n: int) -> np.ndarray:
    """n successive xorshift64* outputs as uniform doubles in [0, 1)."""
    st = _U64(seed)
    out = np.empty(n, np.float64)
    L = lib()
    for i in range(n):
        out[i] = (L.orc_rng_next(C.byref(st)) >> 11) * (1.0 / 9007199254740992.0)
    return out


# ---- models ---------------------------------------------------------------

class Model:
    """NCP + VQ-VAE oracle model loaded from .conf / .ncm files."""

    def __init__(self, conf: str, weights: str):
        self.h = lib().orc_model_load(conf.encode(), weights.encode())
        if not self.h:
            raise RuntimeError("orc_model_load failed")
        L = lib()
        self.total = L.orc_total_codes(self.h)
        self.L, self.D, self.in_vocab = L.orc_L(self.h), L.orc_D(self.h), L.orc_in_vocab(self.h)
        self.T, self.maxV = L.orc_ncp_T(self.h), L.orc_ncp_maxV(self.h)

    def generate(self, prefix, l0=None, temp=0.0, top_k=0, top_p=1.0, cfg=0.0, freq=0.0, mu=0.0,
                 adj=(0.0, 0, 1.0), allow=None, seed=0, cap_floats=0):
        prefix = _i(prefix)
        B = prefix.shape[0]
        l0 = None if l0 is None else _i(l0)
        allow = None if allow is None else np.ascontiguousarray(allow, dtype=np.float64)
        codes = np.zeros((B, self.total), np.int32)
        cap = np.zeros((B, cap_floats), np.float32) if cap_floats else None
        lib().orc_ncp_generate(self.h, _p(l0), _p(prefix), B, temp, top_k, top_p, cfg, freq, mu,
                               adj[0], adj[1], adj[2], _p(allow), seed, _p(codes), _p(cap))
        return (codes, cap) if cap_floats else codes

    def z_to_idx(self, z):
        z = _f(z)
        B = z.shape[0]
        idx = np.zeros((B, self.total), np.int32)
        lib().orc_vq_z_to_idx(self.h, _p(z), B, _p(idx))
        return idx

    def idx_to_zhats(self, idx, n_levels):
        idx = _i(idx)
        B = idx.shape[0]
        outs = [np.zeros((B, self.L, self.D), np.float32) for _ in range(n_levels)]
        arr = (_P * n_levels)(*[o.ctypes.data for o in outs])
        lib().orc_vq_idx_to_zhats(self.h, _p(idx), B, arr)
        return outs

    def next_input(self, codes, level, z_hat, Lnext):
        codes = _i(codes)
        B = codes.shape[0]
        z_hat = _f(z_hat).copy()
        x = np.zeros((B, Lnext, self.D), np.float32)
        lib().orc_vq_next_input(self.h, _p(codes), level, _p(z_hat), _p(x), B)
        return z_hat, x

    def idx_to_ncm_input(self, idx, T):
        idx = _i(idx)
        B = idx.shape[0]
        x = np.zeros((B, T, self.D), np.float32)
        lib().orc_vq_idx_to_ncm_input(self.h, _p(idx), B, _p(x))
        return x

    def encode(self, ids):
        ids = _i(ids)
        B = ids.shape[0]
        z = np.zeros((B, self.L, self.D), np.float32)
        lib().orc_vqvae_encode(self.h, _p(ids), _p(z), B)
        return z

    def decode(self, zhat):
        zhat = _f(zhat)
        B = zhat.shape[0]
        lg = np.zeros((B, self.L, self.in_vocab), np.float32)
        lib().orc_vqvae_decode(self.h, _p(zhat), _p(lg), B)
        return lg

    def decode_tokens(self, codes):
        codes = _i(codes)
        B = codes.shape[0]
        tok = np.zeros((B, self.L), np.int32)
        lib().orc_decode_tokens(self.h, _p(codes), B, _p(tok))
        return tok

    def forward(self, x, prefix):
        x, prefix = _f(x), _i(prefix)
        B = x.shape[0]
        lg = np.zeros((B, self.T, self.maxV), np.float32)
        lib().orc_ncp_forward(self.h, _p(x), _p(prefix), _p(lg), B)
        return lg


class LM:
    """GPT-2 / Qwen2 oracle (full recompute per token, as the reference does)."""

    def __init__(self, conf: str, weights: str, qwen: bool):
        self.h = lib().orc_lm_load(conf.encode(), weights.encode(), int(qwen))
        if not self.h:
            raise RuntimeError("orc_lm_load failed")
        self.V = lib().orc_lm_vocab(self.h)

    def logits(self, ids, last_only=False):
        ids = _i(ids)
        T = ids.size
        out = np.zeros((self.V,) if last_only else (T, self.V), np.float32)
        lib().orc_lm_logits(self.h, _p(ids), T, int(last_only), _p(out))
        return out

    def nll(self, ids):
        """mean next-token negative log-likelihood of one window (gpt2_nll / qwen_nll)"""
        ids = _i(ids)
        return float(lib().orc_lm_nll(self.h, _p(ids), ids.size))

    def generate(self, prompt, n_new, temp=0.0, top_k=0, top_p=1.0, seed=0, eos=-1):
        prompt = _i(prompt)
        out = np.zeros(n_new, np.int32)
        n = lib().orc_lm_generate(self.h, _p(prompt), prompt.size, n_new, temp, top_k, top_p, seed,
                                  eos, _p(out))
        return out[:n]


def safetensors_import_rules(path: str, conv1d_transpose: bool) -> "dict[str, np.ndarray]":
    """What the reference's offline converters make of a .safetensors file (tools/gpt2import.c:385-417,
    tools/qwenimport.c:383-420): F16 / BF16 widened to float32, buffers named "*.attn.bias" dropped, and for GPT-2
    the 2-D c_attn / c_proj / c_fc "*.weight" matrices transposed. Test infrastructure."""
    import json
    import struct
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = raw[8 + hlen:]
    out = {}
    for name, e in header.items():
        if name == "__metadata__" or name.endswith(".attn.bias"):
            continue
        a, b = e["data_offsets"]
        if e["dtype"] == "F32":
            x = np.frombuffer(data[a:b], np.float32)
        elif e["dtype"] == "F16":
            # f16_to_f32 of the converters (gpt2import.c:250-259): normal numbers, infinities and NaNs as IEEE; a
            # subnormal with mantissa m becomes the float whose BITS are 0x33800000 + (m << 13), which equals
            # m * 2^-24 only for m = 1 -- kept, because the .ncm files the reference runs on hold these values
            h = np.frombuffer(data[a:b], np.uint16).astype(np.uint32)
            sg, ex, m = (h >> 15) & 1, (h >> 10) & 0x1F, h & 0x3FF
            bits = np.where(ex == 0, np.where(m != 0, 0x33800000 + (m << 13), 0),
                            np.where(ex == 31, 0x7F800000 | (m << 13), ((ex + 112) << 23) | (m << 13)))
            x = ((sg << 31) | bits).astype(np.uint32).view(np.float32)
        elif e["dtype"] == "BF16":
            x = (np.frombuffer(data[a:b], np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            raise ValueError(e["dtype"])
        x = x.reshape(e["shape"])
        if conv1d_transpose and x.ndim == 2 and name.endswith(".weight") and \
                any(k in name for k in ("c_attn", "c_proj", "c_fc", "proj")):
            x = np.ascontiguousarray(x.T)
        out[name] = np.ascontiguousarray(x, np.float32)
    return out
