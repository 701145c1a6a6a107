"""The reference's own command-line front end, linked against libncm_b200.so, beside the reference's CPU build.

oracle/Makefile's `cli` target compiles the reference's main.c, tok.c and tok_tables.c unchanged, adds the library's
link-time stand-ins for the training / viewer entry points (saphira-cncm_b200/cli_stubs.c) and links them against
the GPU library; `ref` builds the all-CPU binary from the same main.c. Both are run on the same seeded model files
and their output is compared: the text of `gen`, the `idx:` line and stage checksums of `infer`, the per-board
records of `eval-sudoku`, the event stream of `sudoku-stream`, the `ids:` line of `gpt2-gen` / `qwen-gen` and the
`docs=... nll=...` line of `gpt2-ppl`. This is the drop-in boundary exercised the way a user of the reference
would: same commands, same files, the compute objects swapped."""
import dataclasses
import json
import os
import re
import subprocess

import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu

REF_DIR = os.path.dirname(helpers.REF_LIB)
CPU, GPU = os.path.join(REF_DIR, "cncm"), os.path.join(REF_DIR, "cncm_b200")


def _run(exe, args, cwd):
    r = subprocess.run([exe] + args, capture_output=True, text=True, timeout=600, cwd=cwd)
    return r.returncode, r.stdout, r.stderr


@pytest.fixture(scope="module")
def both(tmp_path_factory):
    if not (os.path.exists(CPU) and os.path.exists(GPU)):
        pytest.skip("linked command-line binaries not built (make -C oracle ref cli)")
    return str(tmp_path_factory.mktemp("cli"))


def _sudoku_model(tmp):
    import synth
    # a 9 x 9 board in the reference's framing: wrap | 9 cells (sep 9 cells) x 8 | wrap = 91 ids, ids 0..11
    spec = dataclasses.replace(synth.spec_c1(ladder=(1, 3, 9, 91)), name="cli_sudoku", prefix_len=91)
    conf, w = synth.write_ncp(spec, tmp)
    rng = np.random.default_rng(3)
    rows = []
    for _ in range(5):
        cells = rng.integers(1, 10, size=(9, 9)) * (rng.random((9, 9)) < 0.5)
        ids = [11]
        for r in range(9):
            ids += [int(v) for v in cells[r]]
            if r < 8:
                ids.append(10)
        ids.append(11)
        rows.append(ids)
    return spec, conf, w, rows


def _floats_close(a, b, tol):
    fa, fb = re.findall(r"-?\d+\.\d+", a), re.findall(r"-?\d+\.\d+", b)
    assert len(fa) == len(fb), (a, b)
    for x, y in zip(fa, fb):
        assert abs(float(x) - float(y)) <= tol * max(1.0, abs(float(y))), (a, b)


def test_gen_and_infer_print_what_the_cpu_build_prints(both):
    spec, conf, w, rows = _sudoku_model(both)
    base = ["--conf", conf, "--weights", w, "--asset-dir", both]
    ids = ",".join(map(str, rows[0]))
    for extra in (["--temp", "0"], ["--temp", "0.8", "--top-k", "5", "--top-p", "0.9", "--seed", "3", "--n", "2"]):
        args = ["gen"] + base + ["--prefix", ids] + extra
        want, got = _run(CPU, args, both), _run(GPU, args, both)
        assert want[0] == 0 and got[0] == 0, (want, got)
        assert got[1] == want[1] and want[1].strip(), (extra, got[1], want[1])
    args = ["infer"] + base + ["--ids", ",".join(map(str, rows[1]))]
    want, got = _run(CPU, args, both), _run(GPU, args, both)
    assert want[0] == 0 and got[0] == 0, (want, got)
    wl, gl = want[1].strip().splitlines(), got[1].strip().splitlines()
    assert len(wl) == len(gl) and len(wl) >= 4
    for a, b in zip(gl, wl):
        assert a.split()[0] == b.split()[0]
        if b.startswith("idx:"):
            assert a == b                                  # quantizer codes: exact
        else:
            _floats_close(a, b, 2e-4)                      # checksums printed with six decimals


def test_eval_sudoku_and_stream_records(both):
    spec, conf, w, rows = _sudoku_model(both)
    base = ["--conf", conf, "--weights", w, "--asset-dir", both]
    inp, refs = os.path.join(both, "inputs.txt"), os.path.join(both, "refs.txt")
    with open(inp, "w") as f, open(refs, "w") as g:
        for r in rows:
            f.write(" ".join(map(str, r)) + "\n")
            g.write(" ".join(map(str, r)) + "\n")
    outs = {}
    for tag, exe in (("cpu", CPU), ("gpu", GPU)):
        jl = os.path.join(both, f"eval_{tag}.jsonl")
        rc, out, err = _run(exe, ["eval-sudoku"] + base + ["--inputs", inp, "--refs", refs, "--jsonl", jl], both)
        assert rc == 0, err
        recs = [json.loads(ln) for ln in open(jl)]
        for r in recs:
            r.pop("ms")                                    # wall-clock per board
        outs[tag] = (out, recs)
    assert outs["gpu"][0] == outs["cpu"][0] and "solved" in outs["cpu"][0]
    assert outs["gpu"][1] == outs["cpu"][1] and len(outs["cpu"][1]) == len(rows)
    # the level-by-level event stream (NDJSON) of one board, driven through the stepper API
    args = ["sudoku-stream"] + base + ["--prefix", ",".join(map(str, rows[2])), "--seed", "1"]
    want, got = _run(CPU, args, both), _run(GPU, args, both)
    assert want[0] == got[0] == 0, (want[2], got[2])

    def events(text):
        evs = []
        for ln in text.strip().splitlines():
            e = json.loads(ln)
            for k in [k for k in e if k.endswith("ms") or k in ("t", "elapsed", "time")]:
                e.pop(k)
            evs.append(e)
        return evs
    assert events(got[1]) == events(want[1]) and len(events(want[1])) >= 3


@pytest.mark.parametrize("kind", ["gpt2", "qwen"])
def test_decoder_lm_commands(both, kind):
    import synth
    spec = synth.spec_gpt2_tiny() if kind == "gpt2" else synth.spec_qwen_tiny()
    conf, w = synth.write_lm(spec, both)
    base = ["--conf", conf, "--weights", w, "--asset-dir", both]
    pr = ",".join(str(int(v)) for v in synth.lm_prompts(spec, 1, 9, 3)[0])
    for extra in (["--n", "12"], ["--n", "12", "--temp", "0.7", "--top-p", "0.95", "--seed", "9"]):
        args = [f"{kind}-gen"] + base + ["--ids", pr] + extra
        want, got = _run(CPU, args, both), _run(GPU, args, both)
        assert want[0] == 0 and got[0] == 0, (want, got)
        assert got[1].splitlines()[0] == want[1].splitlines()[0] and want[1].startswith("ids:"), (got[1], want[1])
    # likelihood of a texts file (the configuration's character tokenizer turns the digits into ids on the host)
    texts = os.path.join(both, f"{kind}_texts.txt")
    with open(texts, "w") as f:
        # documents stay inside the tiny models' 64-token context (the reference reads past its rotary table beyond it)
        f.write("123456789|987654321\n5555|1234|99\n\n3\n" + "|".join(["918273645"] * 6) + "\n")
    args = [f"{kind}-ppl"] + base + ["--texts", texts]
    want, got = _run(CPU, args, both), _run(GPU, args, both)
    assert want[0] == 0 and got[0] == 0, (want, got)
    fw = dict(kv.split("=") for kv in want[1].split())
    fg = dict(kv.split("=") for kv in got[1].split())
    assert fg["docs"] == fw["docs"] and fg["tokens"] == fw["tokens"] and int(fw["tokens"]) > 50, (got[1], want[1])
    assert abs(float(fg["nll"]) - float(fw["nll"])) < 1e-4, (got[1], want[1])


def _write_nctrain(path, rows):
    import struct
    rows = np.ascontiguousarray(rows, np.int32)
    with open(path, "wb") as f:
        f.write(b"NCMT" + struct.pack("<QQ", rows.shape[0], rows.shape[1]))
        f.write(rows.tobytes())


def _grid_model(tmp, n, name):
    """an n x n board in the reference's framing: wrap | n cells (sep n cells) x (n-1) | wrap, ids 0..11"""
    import synth
    T = n * n + (n - 1) + 2
    spec = dataclasses.replace(synth.spec_c1(ladder=(1, 3, T)), name=name, prefix_len=T)
    conf, w = synth.write_ncp(spec, tmp)
    rng = np.random.default_rng(5)
    rows = []
    for _ in range(5):
        cells = rng.integers(1, 10, size=(n, n)) * (rng.random((n, n)) < 0.6)
        ids = [11]
        for r in range(n):
            ids += [int(v) for v in cells[r]]
            if r < n - 1:
                ids.append(10)
        ids.append(11)
        rows.append(ids)
    return spec, conf, w, rows


def test_eval_magic_records(both):
    spec, conf, w, rows = _grid_model(both, 3, "cli_magic")
    base = ["--conf", conf, "--weights", w, "--asset-dir", both]
    inp, refs = os.path.join(both, "magic_inputs.txt"), os.path.join(both, "magic_refs.txt")
    with open(inp, "w") as f, open(refs, "w") as g:
        for r in rows:
            f.write(" ".join(map(str, r)) + "\n")
            g.write("".join(str(v) if v else "." for v in r if v < 10)[:9].ljust(9, ".") + "\n")
    outs = {}
    for tag, exe in (("cpu", CPU), ("gpu", GPU)):
        jl = os.path.join(both, f"magic_{tag}.jsonl")
        rc, out, err = _run(exe, ["eval-magic"] + base + ["--inputs", inp, "--refs", refs, "--size", "3", "--jsonl", jl], both)
        assert rc == 0, err
        recs = [json.loads(ln) for ln in open(jl)]
        for r in recs:
            r.pop("ms")
        outs[tag] = (out, recs)
    assert outs["gpu"][0] == outs["cpu"][0] and "solved" in outs["cpu"][0]
    assert outs["gpu"][1] == outs["cpu"][1] and len(outs["cpu"][1]) == len(rows)


def test_vq_encode_and_vq_recon_on_training_rows(both):
    """The two data-preparation commands: rows of ids from NCMT files through the encoder and the quantizer
    (vq-encode writes [prefix | codes] rows) and back through the decoder (vq-recon writes one board per line)."""
    # vq-recon wants a context of n*n + n - 1 ids: 11 for a 3 x 3 grid
    import synth
    spec = dataclasses.replace(synth.spec_c1(ladder=(1, 3, 11)), name="cli_vq", prefix_len=7)
    conf, w = synth.write_ncp(spec, both)
    rng = np.random.default_rng(9)
    nrows = 37                                             # more than one batch of 32
    sol = rng.integers(0, 12, size=(nrows, 11))
    pre = rng.integers(0, 12, size=(nrows, 7))
    ps, pp = os.path.join(both, "sol.nctrain"), os.path.join(both, "pre.nctrain")
    _write_nctrain(ps, sol)
    _write_nctrain(pp, pre)
    base = ["--conf", conf, "--weights", w]
    res = {}
    for tag, exe in (("cpu", CPU), ("gpu", GPU)):
        oe, orc_ = os.path.join(both, f"enc_{tag}.nctrain"), os.path.join(both, f"recon_{tag}.txt")
        rc, out, err = _run(exe, ["vq-encode"] + base + ["--prefix", pp, "--sol", ps, "--out", oe], both)
        assert rc == 0, err
        rc2, out2, err2 = _run(exe, ["vq-recon"] + base + ["--sol", ps, "--out", orc_, "--max-rows", "35"], both)
        assert rc2 == 0, err2
        res[tag] = (open(oe, "rb").read(), out.splitlines()[-1], open(orc_).read(), out2.splitlines()[-1])
    assert res["gpu"][0] == res["cpu"][0]                  # [prefix | codes] rows: bytes equal
    assert len(res["cpu"][0]) == 20 + nrows * (7 + 15) * 4
    assert res["gpu"][1].startswith("[vq-encode] 37 rows x 22 -> ") and res["cpu"][1].startswith("[vq-encode] 37 rows x 22 -> ")
    assert res["gpu"][2] == res["cpu"][2] and len(res["cpu"][2].splitlines()) == 35
    assert res["gpu"][3] == res["cpu"][3] and "id_match" in res["cpu"][3]
    # a cut file and a wrong magic are refused by the reader, with the reference's messages
    bad = os.path.join(both, "cut.nctrain")
    open(bad, "wb").write(open(ps, "rb").read()[:200])
    for exe in (CPU, GPU):
        rc, out, err = _run(exe, ["vq-recon"] + base + ["--sol", bad, "--out", os.path.join(both, "x.txt")], both)
        assert rc == 1 and "short read" in err
