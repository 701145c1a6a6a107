"""linear_fwd (reference src/ncm.h:146, y = x W^T + b) on every GEMM engine of the library.

Engines 0 (fp32 CUDA cores), 2 (three TF32 MMAs over hi/lo pairs) and 3 (three fp16 MMAs over
prescaled fp16 pairs into one accumulator) must all be fp32-grade against a float64 product;
engine 1 (one TF32 pass) is the fast, coarse option and only has to be TF32-grade.
"""
import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu

# (rows, out features, in features): full tiles, ragged tiles, K tails inside a TMA box,
# K not a multiple of 8 (fp16 rows would break the 16-byte stride rule: engine 3 hands over to 2),
# few rows (CUDA-core weight streaming)
SHAPES = [(128, 128, 64), (256, 256, 512), (1000, 768, 520), (333, 200, 100), (2048, 1024, 2048), (8, 512, 512),
          # the fp16-pair engine picks 64-column tiles for these two (the second with ragged edges), 32-column ones for the third
          (2048, 512, 512), (1100, 520, 192), (64, 768, 128),
          # few rows, long K: K runs as slices on CTAs of their own, a second kernel adds them
          (20, 896, 4864), (64, 768, 3072), (130, 512, 2048)]


@pytest.fixture(scope="module")
def cuda():
    import capi
    lib = capi.NcmLib(helpers.CUDA_LIB)
    yield lib
    lib.ncmb_set_gemm_mode(3)


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_linear_fwd_on_every_engine(cuda, shape):
    M, N, K = shape
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    # activations with a wide dynamic range: most entries O(1), some tiny, some in the hundreds
    x = (rng.standard_normal((M, K)) * np.exp(rng.uniform(-9, 5, size=(M, 1)))).astype(np.float32)
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    want = x.astype(np.float64) @ W.astype(np.float64).T + b
    # scale of one row's products: what an fp32 dot product of that row can resolve
    row_scale = (np.abs(x).astype(np.float64) @ np.abs(W).astype(np.float64).T) + np.abs(b)
    xd, Wd, bd = cuda.to_backend(x), cuda.to_backend(W), cuda.to_backend(b)
    yd = cuda.alloc(M * N)
    for mode, rel in ((0, 2e-6), (2, 4e-6), (3, 2e-6), (1, 2e-3)):
        cuda.ncmb_set_gemm_mode(mode)
        cuda.linear_fwd(xd, Wd, bd, yd, M, N, K)
        cuda.ncmb_sync()
        assert cuda.ncmb_gemm_tc_check() == 0
        y = cuda.to_host(yd, (M, N))
        err = np.abs(y - want) / row_scale
        assert err.max() <= rel, f"engine {mode}: {err.max():.3e} of the row scale"


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
@pytest.mark.parametrize("shape", [(256, 256, 512), (1000, 768, 520), (2048, 1024, 2048), (300, 512, 64)], ids=lambda s: "x".join(map(str, s)))
def test_fp16_pair_engine_at_every_tile_width(cuda, shape, bn, monkeypatch):
    """The fp16-pair engine picks its tile width (32 to 256 columns) from the problem size; here every width is
    forced on small shapes, ragged row tiles and a K tail included, with a residual and a bias."""
    M, N, K = shape
    monkeypatch.setenv("NCM_B200_H3_BN", str(bn))
    rng = np.random.default_rng(M + N + K + bn)
    x = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    want = x.astype(np.float64) @ W.astype(np.float64).T + b
    row_scale = (np.abs(x).astype(np.float64) @ np.abs(W).astype(np.float64).T) + np.abs(b)
    xd, Wd, bd = cuda.to_backend(x), cuda.to_backend(W), cuda.to_backend(b)
    yd = cuda.alloc(M * N)
    cuda.ncmb_set_gemm_mode(3)
    cuda.linear_fwd(xd, Wd, bd, yd, M, N, K)
    cuda.ncmb_sync()
    assert cuda.ncmb_gemm_tc_check() == 0
    err = np.abs(cuda.to_host(yd, (M, N)) - want) / row_scale
    assert err.max() <= 2e-6, f"{bn}-column tiles: {err.max():.3e} of the row scale"


def test_descriptor_cache_eviction_between_the_lookups_of_one_launch(cuda):
    """The TMA descriptor caches start over when full. With the limit at one entry every lookup of a launch evicts
    the one before it (a GEMM fetches four or five descriptors, attention three); results must not change."""
    M, N, K = 300, 256, 192
    rng = np.random.default_rng(77)
    x = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    xd, Wd = cuda.to_backend(x), cuda.to_backend(W)
    yd = cuda.alloc(M * N)
    try:
        for mode in (2, 3):
            cuda.ncmb_set_gemm_mode(mode)
            cuda.ncmb_set_map_cache_limit(4096)
            cuda.linear_fwd(xd, Wd, None, yd, M, N, K)
            want = cuda.to_host(yd, (M, N))
            cuda.ncmb_set_map_cache_limit(1)
            for _ in range(3):
                cuda.linear_fwd(xd, Wd, None, yd, M, N, K)
                assert np.array_equal(cuda.to_host(yd, (M, N)), want), mode
            assert cuda.ncmb_gemm_tc_check() == 0
    finally:
        cuda.ncmb_set_map_cache_limit(4096)
