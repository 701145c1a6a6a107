"""The reference's kernel checksum harness (tests/ktest_kernels.c: 14 lines of sum / max-abs / first four values).

tests/golden/ktest_kernels.txt holds what that program prints when built against the reference's CPU objects
(oracle/Makefile `ktest`, run where the reference's sources are).  Here:

* the CPU oracle reproduces every line from the harness's own input stream (its xorshift generator and the order
  in which it draws buffers), digit for digit;
* where the harness binaries are present, the reference build still prints the committed lines, and -- on a GPU --
  the same program linked against libncm_b200.so prints them within fp32 tolerance.
"""
import os
import re
import subprocess

import numpy as np
import pytest

import helpers
import orc

FIXTURE = os.path.join(helpers.HERE, "golden", "ktest_kernels.txt")
REF_DIR = os.path.dirname(helpers.REF_LIB)


class _Stream:
    """frand() of the harness: xorshift (13, 7, 17) on 64 bits, top 53 bits mapped to [-2, 2) and rounded to float"""

    def __init__(self):
        self.s = 0x12345678

    def mk(self, *shape):
        n = int(np.prod(shape))
        out = np.empty(n, np.float32)
        s, M = self.s, (1 << 64) - 1
        for i in range(n):
            s ^= (s << 13) & M
            s ^= s >> 7
            s ^= (s << 17) & M
            out[i] = np.float32((s >> 11) * (1.0 / 9007199254740992.0) * 4.0 - 2.0)
        self.s = s
        return out.reshape(shape)


def _line(name, y):
    h = np.asarray(y, np.float32).ravel()
    s = 0.0
    for v in h:                                   # the harness adds in index order, in double
        s += float(v)
    return "%s sum=%.6f maxabs=%.6f first=%.6f %.6f %.6f %.6f" % (name, s, float(np.abs(h).max()), h[0], h[1], h[2], h[3])


def _oracle_lines():
    r, out = _Stream(), []
    x, w, b, _ = r.mk(4, 64), r.mk(64), r.mk(64), r.mk(4 * 64)
    out.append(_line("layernorm", orc.layernorm(x, w, b)))
    x, w, _ = r.mk(4, 64), r.mk(64), r.mk(4 * 64)
    out.append(_line("rmsnorm", orc.rmsnorm(x, w)))
    x, _ = r.mk(512), r.mk(512)
    out += [_line("gelu", orc.gelu(x)), _line("silu", orc.silu(x)), _line("softmax", orc.softmax(x.reshape(8, 64)))]
    q, k = r.mk(1, 2, 16, 32), r.mk(1, 2, 16, 32)
    co, si = r.mk(16, 32), r.mk(16, 32)
    out += [_line("rope_q", orc.rope(q, co, si, 16)), _line("rope_k", orc.rope(k, co, si, 16))]
    q, k, v, m, _ = r.mk(1, 2, 8, 16), r.mk(1, 2, 12, 16), r.mk(1, 2, 12, 16), r.mk(8, 12), r.mk(1 * 2 * 8 * 16)
    m = np.where(m > 0, 0.0, -np.inf).astype(np.float32)
    out.append(_line("sdpa", orc.sdpa(q, k, v, m)))
    x, W, b, _ = r.mk(2, 4, 32), r.mk(4, 4, 3), r.mk(4), r.mk(2 * 4 * 32)
    out.append(_line("conv1d", orc.conv1d(x, W, b, 1, 1)))
    out.append(_line("groupnorm", orc.groupnorm(x, 4)))
    out.append(_line("area", orc.interp_area(x, 9)))
    # the harness reads the same buffer as [2][4][9] for the linear up-sampling
    out.append(_line("linear_interp", orc.interp_linear(x.ravel()[:2 * 4 * 9].reshape(2, 4, 9), 32)))
    a, bb, _ = r.mk(16, 32), r.mk(8, 32), r.mk(16 * 8)
    out.append(_line("l2sq", orc.l2sq(a, bb)))
    x, W, b, _ = r.mk(8, 64), r.mk(128, 64), r.mk(128), r.mk(8 * 128)
    out.append(_line("linear", orc.linear(x, W, b)))
    return out


def _fixture_lines():
    return [ln for ln in open(FIXTURE).read().splitlines() if ln and ln != "KTEST-DONE"]


def test_oracle_reproduces_the_harness_lines_digit_for_digit():
    want = _fixture_lines()
    assert len(want) == 14
    got = _oracle_lines()
    for g, w in zip(got, want):
        assert g.replace("-0.000000", "0.000000") == w.replace("-0.000000", "0.000000")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_DIR, "ktest_ref")), reason="harness not built (make -C oracle ktest)")
def test_reference_build_prints_the_committed_lines():
    out = subprocess.run([os.path.join(REF_DIR, "ktest_ref")], capture_output=True, text=True, timeout=120).stdout
    assert out.splitlines()[:14] == _fixture_lines() and "KTEST-DONE" in out


@pytest.mark.gpu
def test_harness_linked_against_the_gpu_library_prints_the_same_checksums():
    exe = os.path.join(REF_DIR, "ktest_b200")
    if not os.path.exists(exe):
        pytest.skip("harness not built (make -C oracle ktest)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "KTEST-DONE" in r.stdout, r.stderr[-2000:]
    got, want = r.stdout.splitlines()[:14], _fixture_lines()
    num = re.compile(r"-?\d+\.\d+")
    for g, w in zip(got, want):
        assert g.split()[0] == w.split()[0]
        fg, fw = [float(v) for v in num.findall(g)], [float(v) for v in num.findall(w)]
        assert len(fg) == len(fw) == 6
        n = {"linear": 1024, "l2sq": 128}.get(w.split()[0], 512)
        # sum of n values each good to 2e-5 of the largest magnitude; single values to 2e-5 of their scale
        assert abs(fg[0] - fw[0]) <= 2e-5 * n * max(1.0, fw[1]) * 0.1 + 2e-6, (g, w)
        for a, b in zip(fg[1:], fw[1:]):
            assert abs(a - b) <= 2e-5 * max(1.0, fw[1]) + 1e-6, (g, w)
