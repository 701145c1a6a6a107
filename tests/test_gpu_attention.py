"""Token-major attention of the transformer blocks: the tcgen05 kernel against the CUDA-core kernel
and against a float64 softmax(QK^T/sqrt(d))V, through ncmb_attention_check.

Shapes follow the callers: ragged prefix rows attending to themselves (the NCP prefix pass,
reference src/ncp.c forward over the prefix), causal rows (decoder-LM prefill), rows whose few
queries see a cached segment plus their own tokens (NCP level passes; grouped-query heads are
packed into one tile), and the windowed form of the VQ-VAE attention layers.
"""
import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    import capi
    return capi.NcmLib(helpers.CUDA_LIB)


def _want(q, kv1, kv2, qs, k1s, k2s, H, Hkv, causal, window):
    out = np.zeros(q.shape, dtype=np.float64)
    kvd = Hkv * 64
    for r in range(len(qs) - 1):
        for h in range(H):
            kvh = h // (H // Hkv)
            Q = q[qs[r]:qs[r + 1], h * 64:(h + 1) * 64].astype(np.float64)
            K = kv1[k1s[r]:k1s[r + 1], kvh * 64:(kvh + 1) * 64]
            V = kv1[k1s[r]:k1s[r + 1], kvd + kvh * 64:kvd + (kvh + 1) * 64]
            n1 = K.shape[0]
            if k2s is not None:
                K = np.concatenate([K, kv2[k2s[r]:k2s[r + 1], kvh * 64:(kvh + 1) * 64]])
                V = np.concatenate([V, kv2[k2s[r]:k2s[r + 1], kvd + kvh * 64:kvd + (kvh + 1) * 64]])
            S = Q @ K.astype(np.float64).T * 0.125
            qi = np.arange(Q.shape[0])[:, None]
            kj = np.arange(K.shape[0])[None, :]
            vis = np.ones(S.shape, bool)
            if causal:
                vis &= ~((kj < n1) & (kj > qi))
            if window > 0:
                vis &= np.abs(kj - qi) <= window
            S = np.where(vis, S, -np.inf)
            P = np.exp(S - S.max(1, keepdims=True))
            out[qs[r]:qs[r + 1], h * 64:(h + 1) * 64] = (P / P.sum(1, keepdims=True)) @ V.astype(np.float64)
    return out


CASES = {
    # name: (query rows, segment-1 keys, segment-2 keys or None, H, Hkv, causal, window)
    "one_full_tile": ([128], [128], None, 1, 1, 0, 0),
    "ragged_prefix_rows": ([256, 70, 131, 1], [256, 70, 131, 1], None, 8, 8, 0, 0),
    "grouped_heads_prefix": ([200, 33], [200, 33], None, 8, 2, 0, 0),
    "causal_prefill": ([200, 64, 288], [200, 64, 288], None, 4, 2, 1, 0),
    "grouped_heads_c2_prefix_shape": ([256, 1, 256, 1, 190], [256, 1, 256, 1, 190], None, 8, 2, 0, 0),
    "grouped_heads_16q_4kv": ([256, 100], [256, 100], None, 16, 4, 0, 0),
    "cache_plus_own_tokens": ([32, 17, 24], [250, 3, 77], [32, 17, 24], 4, 4, 0, 0),
    "level_pass_packed_g4": ([32, 17, 1, 4], [250, 3, 77, 256], [32, 17, 1, 4], 8, 2, 0, 0),
    "level_pass_packed_g2": ([16, 5], [40, 100], [16, 5], 4, 2, 0, 0),
    "packed_one_segment_all_288_keys": ([8, 32], [288, 129], None, 4, 1, 0, 0),
    "windowed": ([150], [150], None, 2, 2, 0, 16),
    # rows with more keys than one launch keeps resident: 256-key blocks through the same kernel, then a merge
    "long_causal_prefill_blocks": ([512, 300, 700, 64], [512, 300, 700, 64], None, 4, 2, 1, 0),
    "long_bidirectional_blocks": ([130, 64], [1000, 289], None, 2, 1, 0, 0),
}


@pytest.mark.parametrize("grouping", ["chosen", "kv_group_per_cta"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_tensor_core_attention_matches_cuda_core_and_float64(cuda, name, grouping, monkeypatch):
    qlens, k1lens, k2lens, H, Hkv, causal, window = CASES[name]
    if grouping == "kv_group_per_cta":
        # one CTA walks all heads that share a kv head (what large batches get): keys and values are fetched and
        # converted once, the heads' phases overlap
        if H == Hkv:
            pytest.skip("one head per kv head: nothing to group")
        monkeypatch.setenv("NCM_B200_ATTN_HPC", str(H // Hkv))
    else:
        monkeypatch.delenv("NCM_B200_ATTN_HPC", raising=False)
    rng = np.random.default_rng(sum(map(ord, name)))
    off = lambda lens: np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    qs, k1s = off(qlens), off(k1lens)
    k2s = None if k2lens is None else off(k2lens)
    q = rng.standard_normal((qs[-1], H * 64)).astype(np.float32)
    kv1 = rng.standard_normal((k1s[-1], 2 * Hkv * 64)).astype(np.float32)
    kv2 = None if k2s is None else rng.standard_normal((k2s[-1], 2 * Hkv * 64)).astype(np.float32)
    qd, k1d = cuda.to_backend(q), cuda.to_backend(kv1)
    k2d = None if kv2 is None else cuda.to_backend(kv2)
    want = _want(q, kv1, kv2, qs, k1s, k2s, H, Hkv, causal, window)
    got = {}
    for engine in (0, 1):
        od = cuda.alloc(q.size)
        rc = cuda.ncmb_attention_check(qd, k1d, k2d, od, qs.ctypes.data, k1s.ctypes.data,
                                       None if k2s is None else k2s.ctypes.data,
                                       len(qlens), H, Hkv, causal, window, engine)
        assert rc == 0, (name, engine, rc)
        got[engine] = cuda.to_host(od, q.shape)
    # fp32 CUDA-core kernel: ~1e-6; the fp16-pair products drop only the lo*lo term: a few 1e-6
    assert np.abs(got[0] - want).max() < 4e-6
    assert np.abs(got[1] - want).max() < 8e-6
    assert not np.isnan(got[1]).any()


DECODE_CASES = {
    # one query per row against a cache of ragged lengths: (cache lengths, H, Hkv)
    "gpt2_like_12_heads": ([1, 31, 32, 33, 300, 1000], 12, 12),
    "qwen_like_7_heads_per_kv": ([5, 64, 513, 2048], 14, 2),
    "single_head_group_of_4": ([129, 7], 4, 1),
    # many rows: a CTA walks several 32-key chunks with a running maximum (640 row/kv-head pairs, up to 10 chunks)
    "many_rows_several_chunks_per_cta": (list(np.random.default_rng(1).integers(1, 300, 320)) + [320, 289], 8, 2),
    # enough rows to fill the GPU without splitting keys: one CTA sees all keys of its row and writes the context itself
    "one_cta_per_row_no_merge": (list(np.random.default_rng(2).integers(1, 100, 1300)), 4, 2),
}


@pytest.fixture(params=["chosen", "warp_per_chunk", "tensor_core_rows"])
def decode_kernel(request):
    """the split-key path as dispatched, with the warp-per-chunk kernel forced for every shape it takes, and with the
    kernel that makes the (query, head) pairs of a kv group the 16 rows of an mma.sync tile forced likewise"""
    import os
    if request.param == "warp_per_chunk":
        os.environ["NCM_B200_ATTN_DEC_WARP"] = "1"
    if request.param == "tensor_core_rows":
        os.environ["NCM_B200_ATTN_DEC_MMA"] = "1"
    else:
        os.environ["NCM_B200_ATTN_DEC_MMA"] = "0"
    yield request.param
    os.environ.pop("NCM_B200_ATTN_DEC_WARP", None)
    os.environ.pop("NCM_B200_ATTN_DEC_MMA", None)


def _decode_tol(kernel):
    # fp32 multiply-adds: 4e-6; three TF32 MMAs per product and SFU exponentials, like the tcgen05 kernel: 8e-6
    return 8e-6 if kernel == "tensor_core_rows" else 4e-6


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_split_key_decode_attention_matches_cuda_core_and_float64(cuda, name, decode_kernel):
    lens, H, Hkv = DECODE_CASES[name]
    rng = np.random.default_rng(sum(map(ord, name)))
    rows = len(lens)
    qs = np.arange(rows + 1, dtype=np.int32)
    ks = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    q = rng.standard_normal((rows, H * 64)).astype(np.float32)
    kv = rng.standard_normal((ks[-1], 2 * Hkv * 64)).astype(np.float32)
    want = _want(q, kv, None, qs, ks, None, H, Hkv, 0, 0)
    qd, kd = cuda.to_backend(q), cuda.to_backend(kv)
    got = {}
    for engine in (0, 2):
        od = cuda.alloc(q.size)
        rc = cuda.ncmb_attention_check(qd, kd, None, od, qs.ctypes.data, ks.ctypes.data, None, rows, H, Hkv, 0, 0, engine)
        assert rc == 0, (name, engine, rc)
        got[engine] = cuda.to_host(od, q.shape)
    assert np.abs(got[0] - want).max() < 4e-6
    assert np.abs(got[2] - want).max() < _decode_tol(decode_kernel)
    # twice in a row: the kernel's completion counters must be back at zero after each launch
    od = cuda.alloc(q.size)
    assert cuda.ncmb_attention_check(qd, kd, None, od, qs.ctypes.data, ks.ctypes.data, None, rows, H, Hkv, 0, 0, 2) == 0
    assert np.array_equal(cuda.to_host(od, q.shape), got[2])


def test_split_key_attention_with_a_few_queries_and_two_key_segments(cuda, decode_kernel):
    # the first NCP levels: 1 or 4 new tokens per row attend to the cached prefix and to themselves
    rng = np.random.default_rng(77)
    qlens, k1lens, H, Hkv = [1, 4, 3, 4], [250, 3, 77, 1], 8, 2
    off = lambda lens: np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    qs, k1s, k2s = off(qlens), off(k1lens), off(qlens)
    q = rng.standard_normal((qs[-1], H * 64)).astype(np.float32)
    kv1 = rng.standard_normal((k1s[-1], 2 * Hkv * 64)).astype(np.float32)
    kv2 = rng.standard_normal((k2s[-1], 2 * Hkv * 64)).astype(np.float32)
    want = _want(q, kv1, kv2, qs, k1s, k2s, H, Hkv, 0, 0)
    qd, k1d, k2d = cuda.to_backend(q), cuda.to_backend(kv1), cuda.to_backend(kv2)
    od = cuda.alloc(q.size)
    rc = cuda.ncmb_attention_check(qd, k1d, k2d, od, qs.ctypes.data, k1s.ctypes.data, k2s.ctypes.data, len(qlens), H, Hkv, 0, 0, 2)
    assert rc == 0
    assert np.abs(cuda.to_host(od, q.shape) - want).max() < _decode_tol(decode_kernel)


def test_shapes_outside_the_tensor_core_kernel_are_reported_not_rerouted(cuda):
    # a launch keeps at most 288 padded keys of a row resident, longer rows go through key blocks -- but not with a
    # window mask, which the block form does not take
    qs = np.array([0, 64], np.int32)
    ks = np.array([0, 480], np.int32)
    q = cuda.alloc(64 * 64)
    kv = cuda.alloc(480 * 128)
    out = cuda.alloc(64 * 64)
    assert cuda.ncmb_attention_check(q, kv, None, out, qs.ctypes.data, ks.ctypes.data, None, 1, 1, 1, 0, 16, 1) == -1
