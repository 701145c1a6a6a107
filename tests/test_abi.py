"""CPU-side checks of the drop-in boundary: the shared library loads without a GPU,
exports every symbol the public header declares, lays out the public structs like
the reference does, and parses .conf files to the same bytes."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

import helpers

ROOT = helpers.ROOT
HEADER = os.path.join(ROOT, "include", "ncm_b200.h")
import orc  # noqa: E402

REF_HEADER = os.path.join(orc.reference_dir() or "", "src", "ncm.h")   # absent off the build machine: those checks skip


def _declared():
    src = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r"\b([a-z_0-9]+)\s*\([^;{]*\)\s*;", src)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(helpers.CUDA_LIB):
        import importlib.util
        spec = importlib.util.spec_from_file_location("b200_build", os.path.join(ROOT, "saphira-cncm_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return C.CDLL(helpers.CUDA_LIB, mode=os.RTLD_LOCAL | os.RTLD_NOW)


def test_library_exports_every_declared_symbol(lib):
    names = _declared()
    assert len(names) > 90
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_reference_entry_points_are_all_present(lib):
    # the inference surface a host written against the reference binds
    for n in ("weights_load", "config_load", "arena_init_default", "vqvae_load", "ncp_load", "ncp_generate",
              "ncp_gen_begin", "ncp_gen_step", "ncp_gen_finish", "ncp_gen_abort", "vq_idx_to_zhats",
              "vqvae_decode", "vq_z_to_idx", "vqvae_encode_z", "ncp_forward", "gpt2_cmd_gen", "qwen_cmd_gen",
              "gpt2_cmd_ppl", "gpt2_cmd_verify", "qwen_cmd_ppl", "qwen_cmd_verify",
              "linear_fwd", "sdpa_fwd_gqa", "rowwise_l2sq", "sample_topkp", "argmax_row"):
        assert hasattr(lib, n), n


_PROBE = r"""
#include <stdio.h>
#include <stddef.h>
#include "%s"
int main(void) {
    printf("%%zu %%zu %%zu %%zu ", sizeof(Tensor), sizeof(NamedTensor), sizeof(WeightStore), sizeof(NCMConfig));
    printf("%%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu %%zu\n", offsetof(NCMConfig, n_layer), offsetof(NCMConfig, vocab_size),
           offsetof(NCMConfig, rope_theta), offsetof(NCMConfig, n_kv_heads), offsetof(NCMConfig, vq_embed_dim),
           offsetof(NCMConfig, vq_soft_tau), offsetof(NCMConfig, levels), offsetof(NCMConfig, quant_resi_ratio),
           offsetof(NCMConfig, pre_tok), offsetof(NCMConfig, gen_adj_d));
    return 0;
}
"""


def _probe(header, tmp_path, tag):
    src = tmp_path / f"probe_{tag}.c"
    exe = tmp_path / f"probe_{tag}"
    src.write_text(_PROBE % header)
    subprocess.check_call(["/usr/bin/gcc", "-std=c11", "-o", str(exe), str(src)])
    return subprocess.check_output([str(exe)]).decode().split()


def test_public_structs_compile_as_c_and_have_expected_layout(tmp_path):
    mine = _probe(HEADER, tmp_path, "mine")
    assert mine[0] == "56" and mine[2] == "16"           # Tensor, WeightStore
    if os.path.exists(REF_HEADER):
        assert mine == _probe(REF_HEADER, tmp_path, "ref")


def test_config_load_matches_reference_bytes(lib, tmp_path):
    import cases
    import synth
    lib.config_load.restype = C.c_int
    lib.config_load.argtypes = [C.c_void_p, C.c_char_p]
    size = int(_probe(HEADER, tmp_path, "sz")[3])
    specs = [cases.ncp_spec(v) for v in cases.NCP_VARIANTS] + [synth.spec_c1(), synth.spec_c2()]
    ref = None
    if os.path.exists(helpers.REF_LIB):
        ref = C.CDLL(helpers.REF_LIB, mode=os.RTLD_LOCAL)
        ref.config_load.restype = C.c_int
        ref.config_load.argtypes = [C.c_void_p, C.c_char_p]
    for spec in specs:
        conf = str(tmp_path / f"{spec.name}.conf")
        synth.write_conf(conf, synth.ncp_conf(spec))
        a = C.create_string_buffer(size)
        assert lib.config_load(a, conf.encode()) == 0
        got = np.frombuffer(a.raw, np.uint8)
        # spot-check decoded fields
        n_layer = np.frombuffer(a.raw[64:68], np.int32)[0]
        assert n_layer == spec.n_layer
        if ref is not None:
            b = C.create_string_buffer(size)
            assert ref.config_load(b, conf.encode()) == 0
            assert (got == np.frombuffer(b.raw, np.uint8)).all(), spec.name
    for lmspec in (synth.spec_gpt2_124m(), synth.spec_qwen_05b()):
        conf = str(tmp_path / f"{lmspec.name}.conf")
        synth.write_conf(conf, synth.lm_conf(lmspec))
        a = C.create_string_buffer(size)
        assert lib.config_load(a, conf.encode()) == 0
        if ref is not None:
            b = C.create_string_buffer(size)
            assert ref.config_load(b, conf.encode()) == 0
            assert a.raw == b.raw, lmspec.name
    assert lib.config_load(C.create_string_buffer(size), b"/nonexistent/x.conf") == -1


def test_host_side_helpers_match_oracle(lib):
    import orc
    lib.rng_next.restype = C.c_ulonglong
    lib.rng_next.argtypes = [C.POINTER(C.c_ulonglong)]
    lib.sample_topkp.restype = C.c_int
    lib.sample_topkp.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_float, C.POINTER(C.c_ulonglong)]
    lib.argmax_row.restype = C.c_int
    lib.argmax_row.argtypes = [C.c_void_p, C.c_int]
    rng = np.random.default_rng(1)
    st, ost = C.c_ulonglong(77), 77
    for i in range(40):
        row = rng.standard_normal(97).astype(np.float32)
        t, tk, tp = [(0.0, 0, 1.0), (0.8, 5, 0.9), (1.0, 0, 0.6), (0.7, 50, 1.0)][i % 4]
        got = lib.sample_topkp(row.ctypes.data, row.size, t, tk, tp, C.byref(st))
        want, ost = orc.sample_topkp(row, t, tk, tp, ost)
        assert got == want and st.value == ost
        assert lib.argmax_row(row.ctypes.data, row.size) == int(row.argmax())


def test_reference_front_end_links_against_the_library():
    """The reference's main.c + tok.c + tok_tables.c, compiled unchanged, link against libncm_b200.so with nothing but
    the library's stand-ins for the training / viewer entry points (oracle/Makefile `cli`): every inference symbol
    the reference's command-line front end uses is exported. (What the linked binary prints is compared with the
    CPU build in tests/test_gpu_cli.py.)"""
    ref_dir = os.path.dirname(helpers.REF_LIB)
    exe, main_o = os.path.join(ref_dir, "cncm_b200"), os.path.join(ref_dir, "main_cli.o")
    if not os.path.exists(main_o):
        pytest.skip("reference sources were not available when the checkers were built")
    assert os.path.exists(exe)
    need = {ln.split()[-1] for ln in subprocess.check_output(["nm", "-u", main_o], text=True).splitlines() if ln.strip()}
    have = set()
    for f in (helpers.CUDA_LIB, os.path.join(ref_dir, "tok.o"), os.path.join(ref_dir, "tok_tables.o"), os.path.join(ref_dir, "cli_stubs.o")):
        flag = ["-D", "--defined-only"] if f.endswith(".so") else ["--defined-only"]
        have |= {ln.split()[-1] for ln in subprocess.check_output(["nm"] + flag + [f], text=True).splitlines() if ln.strip()}
    missing = sorted(s for s in need - have if not s.startswith("_") and "@" not in s and s not in _LIBC)
    assert not missing, missing
    # the stand-ins cover training / viewers only: none of them shadows an inference entry point of the library
    stubs = {ln.split()[-1] for ln in subprocess.check_output(["nm", "--defined-only", os.path.join(ref_dir, "cli_stubs.o")], text=True).splitlines()
             if " T " in ln}
    lib_syms = {ln.split()[-1] for ln in subprocess.check_output(["nm", "-D", "--defined-only", helpers.CUDA_LIB], text=True).splitlines() if ln.strip()}
    assert not (stubs & lib_syms), sorted(stubs & lib_syms)


_LIBC = {"calloc", "clock_gettime", "exit", "fclose", "fflush", "fgets", "fopen", "fputc", "free", "fseek", "ftell", "fwrite", "getenv",
         "malloc", "memcpy", "memset", "omp_set_num_threads", "snprintf", "stderr", "stdin", "stdout", "strchr", "strcmp", "strlen",
         "strncmp", "strtod", "strtol", "strtoll", "strtoull", "printf", "fprintf", "puts", "putchar", "atoi", "atof", "strstr", "qsort",
         "realloc", "fread", "sprintf", "sscanf", "memcmp", "strncpy", "strcpy", "strdup", "exp", "log", "pow", "sqrt", "fputs", "getline",
         "strrchr", "memmove", "abort", "rand", "srand", "time", "floor", "ceil", "fabs", "usleep", "nanosleep", "isatty", "fileno", "read"}
