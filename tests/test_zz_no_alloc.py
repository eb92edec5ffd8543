"""The product entry point that allocates nothing (b200_matmul_f32_static_scratch) against the ordinary
path (a dot_general program compiled and executed through the same C ABI). Collected last so that it also runs
after every other GPU test of the session has used the device; it passes alone in a fresh process as well."""
import numpy as np
import pytest

from b200.shlo.builder import Builder

pytestmark = pytest.mark.gpu


def _dot_text(m, k, n):
    b = Builder()
    a, w = b.arg((m, k), "f32"), b.arg((k, n), "f32")
    return b.module([b.matmul(a, w)])


def _both_ways(client, m, k, n, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32)
    exe = client.compile(_dot_text(m, k, n))
    da, dw = client.buffer_from_host(a), client.buffer_from_host(w)
    want = exe.execute([da, dw])[0].to_numpy()
    out = client.buffer_from_host(np.full((m, n), np.nan, np.float32))
    client.matmul_static_scratch(da, dw, out)
    client.synchronize()
    return out.to_numpy(), want, a, w


def test_two_calls_in_a_row_match_the_compiled_product(client):
    # the second call is smaller and uses fewer splits, so stale partial sums of the first would show
    for seed, (m, k, n) in enumerate([(300, 4096, 200), (64, 200, 48), (1024, 512, 1024)]):
        got, want, a, w = _both_ways(client, m, k, n, seed)
        scale = float(np.max(np.abs(want)))
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5 * max(1.0, scale))
        ref = a.astype(np.float64) @ w.astype(np.float64)
        np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-5 * max(1.0, scale))


def test_same_inputs_twice_give_identical_bits(client):
    g1, _, _, _ = _both_ways(client, 257, 1000, 129, 7)
    g2, _, _, _ = _both_ways(client, 257, 1000, 129, 7)
    np.testing.assert_array_equal(g1, g2)


def test_products_beyond_the_static_scratch_are_refused(client):
    import b200
    a = client.buffer_from_host(np.zeros((2048, 8), np.float32))
    w = client.buffer_from_host(np.zeros((8, 1024), np.float32))
    out = client.buffer_from_host(np.zeros((2048, 1024), np.float32))
    with pytest.raises(b200.B200Error, match="static scratch"):
        client.matmul_static_scratch(a, w, out)


def test_a_call_allocates_no_device_memory(client):
    """After a first call on the device (which loads the library image and looks up the array's address), a call leaves
    the client's allocation counters and the device's free memory where they were."""
    import torch
    rng = np.random.default_rng(11)
    a = client.buffer_from_host(rng.standard_normal((128, 512)).astype(np.float32))
    w = client.buffer_from_host(rng.standard_normal((512, 96)).astype(np.float32))
    out = client.buffer_from_host(np.zeros((128, 96), np.float32))
    client.matmul_static_scratch(a, w, out)             # warm-up
    client.synchronize()
    before, free_before = client.memory_stats(), torch.cuda.mem_get_info(0)[0]
    for _ in range(3):
        client.matmul_static_scratch(a, w, out)
    client.synchronize()
    after, free_after = client.memory_stats(), torch.cuda.mem_get_info(0)[0]
    assert (after.num_allocs, after.bytes_in_use) == (before.num_allocs, before.bytes_in_use)
    assert free_after == free_before
