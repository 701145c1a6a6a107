"""Generates tests/golden/golden.npz from the reference's own CPU build.

Run in a container that has the reference sources:
    make -C oracle ref && python tests/golden/make_golden.py
The reference library (oracle/_ref/libcncm_ref.so) is compiled from the
reference's unmodified sources; this script only calls its public C functions
(src/ncm.h) and two thin wrappers around its file-static GPT-2 / Qwen2 forward
functions (oracle/ref_lm_wrap.c).  Inputs come from seeds (tests/golden/cases.py,
saphira-cncm_b200/synth.py); a SHA-256 of every generated weight file is stored so
a drifting random stream is detected instead of silently mis-compared.
"""
import ctypes as C
import hashlib
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (os.path.join(ROOT, "saphira-cncm_b200"), os.path.join(ROOT, "oracle"), HERE):
    sys.path.insert(0, p)

sys.path.insert(0, os.path.join(ROOT, 'tests'))
import capi      # noqa: E402
import cases     # noqa: E402
import synth     # noqa: E402
from helpers import capi_kernels, capi_ncp, sha  # noqa: E402

REF = os.path.join(ROOT, "oracle", "_ref", "libcncm_ref.so")


def lms(ref, out, tmp):
    I, F, P, U = C.c_int, C.c_float, C.c_void_p, C.c_ulonglong
    for kind, spec in (("gpt2", synth.spec_gpt2_tiny()), ("qwen", synth.spec_qwen_tiny())):
        conf, w = synth.write_lm(spec, tmp)
        out[f"sha_{kind}"] = np.frombuffer(bytes.fromhex(sha(w)), np.uint8)
        cfg = ref.load_config(conf)
        op = getattr(ref.lib, f"ref_{kind}_open"); op.restype = P; op.argtypes = [P, C.c_char_p, C.c_char_p]
        h = op(cfg, w.encode(), tmp.encode())
        assert h
        prompts = synth.lm_prompts(spec, 2, 9, 3)
        for i, pr in enumerate(prompts):
            pr = np.ascontiguousarray(pr)
            lg = np.zeros((pr.size, spec.vocab), np.float32)
            fn = getattr(ref.lib, f"ref_{kind}_logits"); fn.restype = None
            if kind == "gpt2":
                fn.argtypes = [P, P, I, P]; fn(h, pr.ctypes.data, pr.size, lg.ctypes.data)
            else:
                fn.argtypes = [P, P, I, I, P]; fn(h, pr.ctypes.data, pr.size, 0, lg.ctypes.data)
            out[f"lm_{kind}_logits{i}"] = lg
            nl = getattr(ref.lib, f"ref_{kind}_nll"); nl.restype = C.c_double; nl.argtypes = [P, P, I]
            out[f"lm_{kind}_nll{i}"] = np.array([nl(h, pr.ctypes.data, pr.size)], np.float64)
            gen = getattr(ref.lib, f"ref_{kind}_generate"); gen.restype = I
            gen.argtypes = [P, P, I, I, F, I, F, U, P]
            for tag, (t, tk, tp, sd) in (("greedy", (0.0, 0, 1.0, 0)), ("sampled", (0.7, 0, 0.95, 9)), ("topk", (0.9, 8, 1.0, 5))):
                o = np.zeros(12, np.int32)
                n = gen(h, pr.ctypes.data, pr.size, 12, t, tk, tp, sd, o.ctypes.data)
                out[f"lm_{kind}_gen{i}_{tag}"] = o[:n]


def main():
    ref = capi.NcmLib(REF)
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        capi_kernels(ref, out)
        capi_ncp(ref, out, tmp)
        lms(ref, out, tmp)
    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
