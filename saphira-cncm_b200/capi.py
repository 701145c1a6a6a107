"""ctypes binding of the C interface shared by the reference and this library.

The reference has no plugin layer: its boundary is the C symbols of
``src/ncm.h``.  ``libncm_b200.so`` exports the inference part of that header
with identical signatures (declared in ``include/ncm_b200.h``), so one binding
class serves both the CUDA library and the reference's CPU build used as a
checker.  Pointers handed to model functions are *backend* pointers: device
memory for the CUDA library, host memory for a CPU build; ``mem_h2d`` /
``mem_d2h`` move data either way (src/ncm.h:41-46).

``NCMConfig`` is treated as an opaque buffer filled by ``config_load``; only the
library reads its fields.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_I = C.c_int
_F = C.c_float
_P = C.c_void_p
_U64 = C.c_ulonglong
_I64 = C.c_int64
_SZ = C.c_size_t

CONFIG_BYTES = 16384          # generous upper bound on sizeof(NCMConfig) (3.7 KB)


class WeightStore(C.Structure):
    _fields_ = [("items", _P), ("count", _I)]


class Tensor(C.Structure):
    """src/ncm.h:27-34"""
    _fields_ = [("data", _P), ("shape", _I64 * 4), ("ndim", _I), ("n", _I64)]


# name -> (restype, argtypes); only the inference surface
_SIGS = {
    # runtime (src/ncm.h:37-70,139,261)
    "tensor_alloc": (_P, [_I, C.POINTER(_I64)]),
    "tensor_free": (None, [_P]),
    "mem_d2h": (None, [_P, _P, _SZ]),
    "mem_h2d": (None, [_P, _P, _SZ]),
    "mem_d2d": (None, [_P, _P, _SZ]),
    "arena_init": (None, [_SZ]),
    "arena_init_default": (None, []),
    "arena_alloc": (_P, [_SZ]),
    "arena_reset": (None, []),
    "arena_free": (None, []),
    "parena_init": (None, [_SZ]),
    "parena_alloc": (_P, [_SZ]),
    "weights_load": (_I, [C.POINTER(WeightStore), C.c_char_p]),
    "weights_free": (None, [C.POINTER(WeightStore)]),
    "ckpt_probe": (_I, [C.c_char_p]),
    "ckpt_load_weights_only": (_I, [C.c_char_p, C.POINTER(WeightStore), C.c_char_p, _SZ]),
    "weights_get": (_P, [C.POINTER(WeightStore), C.c_char_p]),
    "config_load": (_I, [_P, C.c_char_p]),
    "train_data_load": (_P, [C.c_char_p, _I]),
    "train_data_free": (None, [_P]),
    # layer kernels (src/ncm.h:146-199)
    "linear_fwd": (None, [_P, _P, _P, _P, _I64, _I, _I]),
    "embedding_fwd": (None, [_P, _P, _P, _I64, _I]),
    "layernorm_fwd": (None, [_P, _P, _P, _P, _I64, _I]),
    "layernorm_eps_fwd": (None, [_P, _P, _P, _P, _I64, _I, _F]),
    "rmsnorm_fwd": (None, [_P, _P, _P, _I64, _I]),
    "gelu_fwd": (None, [_P, _P, _I64]),
    "gelu_tanh_fwd": (None, [_P, _P, _I64]),
    "silu_fwd": (None, [_P, _P, _I64]),
    "softmax_fwd": (None, [_P, _P, _I64, _I]),
    "rope_apply": (None, [_P, _P, _P, _P, _I, _I, _I, _I]),
    "rope_apply_gqa": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _I]),
    "heads_transpose_fwd": (None, [_P, _P, _I64, _I, _I]),
    "heads_transpose_fwd_b": (None, [_P, _P, _I, _I64, _I, _I]),
    "sdpa_fwd": (None, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I]),
    "sdpa_fwd_gqa": (None, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I]),
    "conv1d_fwd": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I]),
    "convtranspose1d_fwd": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I]),
    "groupnorm_fwd": (None, [_P, _P, _I, _I, _I, _I]),
    "interpolate_area_fwd": (None, [_P, _P, _I, _I, _I, _I]),
    "interpolate_linear_fwd": (None, [_P, _P, _I, _I, _I, _I]),
    "rowwise_l2sq": (None, [_P, _P, _P, _I64, _I64, _I]),
    "add_fwd": (None, [_P, _P, _P, _I64]),
    "scale_fwd": (None, [_P, _F, _P, _I64]),
    "mul_fwd": (None, [_P, _P, _P, _I64]),
    "add_inplace_fwd": (None, [_P, _P, _I64]),
    "qkv_split_fwd": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I]),
    "head_merge_fwd": (None, [_P, _P, _I, _I, _I, _I, _I]),
    "argmax_row": (_I, [_P, _I]),
    "sample_topkp": (_I, [_P, _I, _F, _I, _F, C.POINTER(_U64)]),
    "rng_next": (_U64, [C.POINTER(_U64)]),
    # models (src/ncm.h:205-287)
    "vqvae_load": (_P, [_P, C.POINTER(WeightStore)]),
    "vqvae_free": (None, [_P]),
    "vqvae_vq": (_P, [_P]),
    "vq_total_codes": (_I, [_P]),
    "vq_z_to_idx": (None, [_P, _P, _I, _P]),
    "vq_idx_to_zhats": (None, [_P, _P, _I, _P]),
    "vq_next_input": (None, [_P, _P, _I, _P, _P, _I]),
    "vq_idx_to_ncm_input": (None, [_P, _P, _I, _P]),
    "vqvae_encode_z": (None, [_P, _P, _P, _I]),
    "vqvae_decode": (None, [_P, _P, _P, _I]),
    "ncp_load": (_P, [_P, C.POINTER(WeightStore), _P]),
    "ncp_free": (None, [_P]),
    "ncp_forward": (None, [_P, _P, _P, _P, _I]),
    "ncp_generate": (_P, [_P, _P, _P, _I, _F, _I, _F, _F, _F, _F, _F, _I, _F, _P, _U64]),
    "ncp_gen_begin": (_P, [_P, _P, _P, _I, _F, _I, _F, _F, _F, _F, _F, _I, _F, _P, _U64]),
    "ncp_gen_step": (_I, [_P, _P, _P]),
    "ncp_gen_finish": (_P, [_P]),
    "ncp_gen_abort": (None, [_P]),
    "ncp_gen_nsteps": (_I, [_P]),
    "ncp_gen_step_size": (_I, [_P, _I]),
    "gpt2_cmd_gen": (_I, [_P, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, _I, _F, _I, _F, _U64]),
    "qwen_cmd_gen": (_I, [_P, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, _I, _F, _I, _F, _U64]),
    # additions of libncm_b200.so (include/ncm_b200.h, "additions")
    "ncmb_version": (C.c_char_p, []),
    "ncmb_set_stream": (None, [_P]),
    "ncmb_get_stream": (_P, []),
    "ncmb_sync": (None, []),
    "ncmb_set_gemm_mode": (None, [_I]),
    "ncmb_get_gemm_mode": (_I, []),
    "ncmb_gemm_tc_check": (_I, []),
    "ncmb_set_lm_persistent": (None, [_I]),
    "ncmb_attention_check": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I]),
    "ncmb_set_rng_mode": (None, [_I]),
    "ncmb_set_row_offset": (None, [C.c_longlong]),
    "ncmb_prof_enable": (None, [_I]),
    "ncmb_prof_reset": (None, []),
    "ncmb_prof_dump_shapes": (None, []),
    "ncmb_prof_top_shape": (_I, [_I, C.POINTER(C.c_longlong), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                 C.POINTER(C.c_double)]),
    "ncmb_prof_read": (_I, [_I, C.POINTER(C.c_longlong), C.POINTER(C.c_double), C.POINTER(C.c_double),
                            C.POINTER(C.c_double)]),
    "ncmb_linear_fwd_noalloc": (_I, [_P, _P, _P, _P, _I64, _I, _I]),
    "ncmb_linear_fwd_noalloc_check": (_I, []),
    "ncmb_set_map_cache_limit": (None, [_I]),
    "ncmb_launch_count": (C.c_longlong, []),
    "ncmb_sample_rows_dev": (None, [_P, _I, _I, _F, _I, _F, _P, _P]),
    "ncmb_forget_weight_copies": (None, []),
    "ncmb_weights_are_bf16": (_I, [C.POINTER(WeightStore)]),
    "ncmb_mem_info": (None, [C.POINTER(_U64), C.POINTER(_U64)]),
    "ncmb_copy_bytes": (None, [C.POINTER(_U64), C.POINTER(_U64)]),
    "ncmb_ncp_generate_ex": (_P, [_P, _P, _P, _I, _F, _I, _F, _F, _F, _F, _F, _I, _F, _P, _U64, _P]),
    "ncmb_decode_tokens": (None, [_P, _P, _I, _P]),
    "ncmb_gen_codes_dev": (_P, [_P]),
    "ncmb_decode_tokens_dev": (None, [_P, _P, _I, _P]),
    "ncmb_vq_encode_dev": (None, [_P, _P, _I, _P]),
    "ncmb_vq_nearest_dev": (None, [_P, _I, _P, C.c_longlong, _P]),
    "ncmb_lm_open": (_P, [_P, C.c_char_p, _I, _I]),
    "ncmb_lm_close": (None, [_P]),
    "ncmb_lm_vocab": (_I, [_P]),
    "ncmb_lm_generate": (_I, [_P, _P, _I, _I, _I, _F, _I, _F, _U64, _I, _P]),
    "ncmb_lm_logits": (None, [_P, _P, _I, _I, _P]),
    "ncmb_lm_nll": (None, [_P, _P, _I, _I, _P, _P]),
    "ncmb_weights_import_safetensors": (_I, [C.POINTER(WeightStore), C.c_char_p, _I]),
    "gpt2_cmd_ppl": (_I, [_P, C.c_char_p, C.c_char_p, C.c_char_p]),
    "gpt2_cmd_verify": (_I, [_P, C.c_char_p, C.c_char_p, C.c_char_p]),
    "qwen_cmd_ppl": (_I, [_P, C.c_char_p, C.c_char_p, C.c_char_p]),
    "qwen_cmd_verify": (_I, [_P, C.c_char_p, C.c_char_p, C.c_char_p]),
}

_libc = C.CDLL(None)
_libc.free.argtypes = [_P]


class NcmLib:
    """One loaded library exporting the ncm.h inference surface."""

    def __init__(self, path: str, extra: "dict[str, tuple] | None" = None):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.path = path
        self.lib = C.CDLL(path, mode=os.RTLD_LOCAL | os.RTLD_NOW)
        sigs = dict(_SIGS)
        if extra:
            sigs.update(extra)
        for name, (res, args) in sigs.items():
            try:
                fn = getattr(self.lib, name)
            except AttributeError:
                continue
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, fn)

    def has(self, name: str) -> bool:
        return hasattr(self, name)

    # ---- small conveniences over backend memory ----
    def to_backend(self, arr: np.ndarray) -> int:
        """Copy a host array into a fresh backend tensor; returns the data pointer.

        The Tensor header is leaked on purpose (test/bench helper)."""
        a = np.ascontiguousarray(arr)
        nfl = (a.nbytes + 3) // 4
        shape = (_I64 * 1)(max(nfl, 1))
        t = self.tensor_alloc(1, shape)
        data = C.cast(t, C.POINTER(_P))[0]
        if a.nbytes:
            self.mem_h2d(data, a.ctypes.data, a.nbytes)
        return data

    def alloc(self, n_floats: int) -> int:
        shape = (_I64 * 1)(max(int(n_floats), 1))
        t = self.tensor_alloc(1, shape)
        return C.cast(t, C.POINTER(_P))[0]

    def to_host(self, ptr: int, shape, dtype=np.float32) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        if out.nbytes:
            self.mem_d2h(out.ctypes.data, ptr, out.nbytes)
        return out

    def load_config(self, conf_path: str):
        buf = C.create_string_buffer(CONFIG_BYTES)
        if self.config_load(buf, conf_path.encode()) != 0:
            raise RuntimeError(f"config_load failed: {conf_path}")
        return buf

    def tensor_host(self, ws: WeightStore, name: str):
        """float32 copy of one named tensor (None if the store has no such name)"""
        p = self.weights_get(C.byref(ws), name.encode())
        if not p:
            return None
        t = C.cast(p, C.POINTER(Tensor)).contents
        out = np.zeros([t.shape[d] for d in range(t.ndim)], np.float32)
        assert out.size == t.n
        if out.size:
            self.mem_d2h(out.ctypes.data, t.data, out.nbytes)
        return out

    def load_weights(self, path: str) -> WeightStore:
        ws = WeightStore()
        if self.weights_load(C.byref(ws), path.encode()) != 0:
            raise RuntimeError(f"weights_load failed: {path}")
        return ws


class NcpModel:
    """config + weights + VQ-VAE + NCP state, as the reference CLI's app_load
    builds them (src/main.c:145-151)."""

    def __init__(self, lib: NcmLib, conf_path: str, weights_path: str, arena_mb: int = 0):
        self.lib = lib
        self.cfg = lib.load_config(conf_path)
        self.ws = lib.load_weights(weights_path)
        if arena_mb:
            lib.arena_init(arena_mb << 20)
        else:
            lib.arena_init_default()
        self.vqvae = lib.vqvae_load(self.cfg, C.byref(self.ws))
        self.ncp = lib.ncp_load(self.cfg, C.byref(self.ws), self.vqvae)
        self.vq = lib.vqvae_vq(self.vqvae)
        self.total = lib.vq_total_codes(self.vq)

    def generate(self, prefix: np.ndarray, l0=None, temp=0.0, top_k=0, top_p=1.0, cfg=0.0,
                 freq=0.0, mu=0.0, adj=(0.0, 0, 1.0), allow=None, seed=0) -> np.ndarray:
        prefix = np.ascontiguousarray(prefix, dtype=np.int32)
        B = prefix.shape[0]
        l0p = None
        if l0 is not None:
            l0 = np.ascontiguousarray(l0, dtype=np.int32)
            l0p = l0.ctypes.data
        ap = None
        if allow is not None:
            allow = np.ascontiguousarray(allow, dtype=np.float64)
            ap = allow.ctypes.data
        out = self.lib.ncp_generate(self.ncp, l0p, prefix.ctypes.data, B, temp, top_k, top_p,
                                    cfg, freq, mu, adj[0], adj[1], adj[2], ap, seed)
        codes = np.ctypeslib.as_array(C.cast(out, C.POINTER(_I)), shape=(B, self.total)).copy()
        _libc.free(out)
        return codes

    def generate_ex(self, prefix: np.ndarray, cap_floats: int, l0=None, temp=0.0, top_k=0, top_p=1.0,
                    cfg=0.0, freq=0.0, mu=0.0, adj=(0.0, 0, 1.0), allow=None, seed=0):
        """libncm_b200 only: codes plus the logits every sampled position was drawn from."""
        prefix = np.ascontiguousarray(prefix, dtype=np.int32)
        B = prefix.shape[0]
        l0p = None
        if l0 is not None:
            l0 = np.ascontiguousarray(l0, dtype=np.int32)
            l0p = l0.ctypes.data
        ap = None
        if allow is not None:
            allow = np.ascontiguousarray(allow, dtype=np.float64)
            ap = allow.ctypes.data
        cap = np.zeros((B, cap_floats), np.float32)
        out = self.lib.ncmb_ncp_generate_ex(self.ncp, l0p, prefix.ctypes.data, B, temp, top_k, top_p, cfg, freq,
                                            mu, adj[0], adj[1], adj[2], ap, seed, cap.ctypes.data)
        codes = np.ctypeslib.as_array(C.cast(out, C.POINTER(_I)), shape=(B, self.total)).copy()
        _libc.free(out)
        return codes, cap

    def decode_tokens(self, codes: np.ndarray, L: int) -> np.ndarray:
        codes = np.ascontiguousarray(codes, dtype=np.int32)
        tok = np.zeros((codes.shape[0], L), np.int32)
        self.lib.ncmb_decode_tokens(self.vqvae, codes.ctypes.data, codes.shape[0], tok.ctypes.data)
        return tok
