"""Threefry-2x32 written as StableHLO integer operations (add, xor, or, shifts on ui32: what jax.random lowers to
without a fused kernel) must be bit-exact. The reference pins its fused Metal kernel against the CPU backend's integers
(tests/configs/random.py:54-74 of the reference); here the checker is an independent NumPy restatement of the
published algorithm (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11), itself held
to that paper's known-answer vectors for 20 rounds."""
import numpy as np
import pytest

import b200
from b200.shlo import programs
from oracle import interp


def _rotl(x, r):
    return ((x << np.uint32(r)) | (x >> np.uint32(32 - r))).astype(np.uint32)


def threefry2x32(k0, k1, x0, x1):
    k0, k1, x0, x1 = (np.asarray(v, np.uint32) for v in (k0, k1, x0, x1))
    with np.errstate(over="ignore"):
        ks = [k0, k1, (k0 ^ k1 ^ np.uint32(0x1BD11BDA)).astype(np.uint32)]
        rot = [(13, 15, 26, 6), (17, 29, 16, 24)]
        x0 = (x0 + ks[0]).astype(np.uint32)
        x1 = (x1 + ks[1]).astype(np.uint32)
        for i in range(5):
            for r in rot[i % 2]:
                x0 = (x0 + x1).astype(np.uint32)
                x1 = _rotl(x1, r) ^ x0
            x0 = (x0 + ks[(i + 1) % 3]).astype(np.uint32)
            x1 = (x1 + ks[(i + 2) % 3] + np.uint32(i + 1)).astype(np.uint32)
    return x0, x1


KNOWN_ANSWERS = [((0x00000000, 0x00000000), (0x00000000, 0x00000000), (0x6B200159, 0x99BA4EFE)),
                 ((0xFFFFFFFF, 0xFFFFFFFF), (0xFFFFFFFF, 0xFFFFFFFF), (0x1CB996FC, 0xBB002BE7)),
                 ((0x13198A2E, 0x03707344), (0x243F6A88, 0x85A308D3), (0xC4923A9C, 0x483DF7A0))]


def test_numpy_restatement_meets_the_known_answers():
    for key, ctr, want in KNOWN_ANSWERS:
        got = threefry2x32(key[0], key[1], ctr[0], ctr[1])
        assert (int(got[0]), int(got[1])) == want


def test_oracle_runs_the_stablehlo_program_bit_exactly():
    prog = programs.threefry_block(3)
    for key, ctr, want in KNOWN_ANSWERS:
        out = interp.run_text(prog.text, [np.array(key, np.uint32), np.array([ctr[0], 1, 2], np.uint32),
                                          np.array([ctr[1], 3, 4], np.uint32)])
        assert (int(out[0][0]), int(out[1][0])) == want
    rng = np.random.default_rng(0)
    prog = programs.threefry_block(257)
    key = rng.integers(0, 1 << 32, 2, dtype=np.uint64).astype(np.uint32)
    x0, x1 = (rng.integers(0, 1 << 32, 257, dtype=np.uint64).astype(np.uint32) for _ in range(2))
    out = interp.run_text(prog.text, [key, x0, x1])
    want = threefry2x32(key[0], key[1], x0, x1)
    np.testing.assert_array_equal(out[0], want[0])
    np.testing.assert_array_equal(out[1], want[1])
    b200.compile_to_plan(prog.text, validate=True)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [3, 1000, 1 << 20])
def test_threefry_on_the_gpu_is_bit_exact(client, n):
    from util import run_gpu
    rng = np.random.default_rng(n)
    key = rng.integers(0, 1 << 32, 2, dtype=np.uint64).astype(np.uint32)
    if n == 3:
        prog = programs.threefry_block(3)
        for k, ctr, want in KNOWN_ANSWERS:
            got, _ = run_gpu(client, prog.text, [np.array(k, np.uint32), np.array([ctr[0], 1, 2], np.uint32),
                                                 np.array([ctr[1], 3, 4], np.uint32)])
            assert (int(got[0][0]), int(got[1][0])) == want
        return
    prog = programs.threefry_bits(n)
    got, _ = run_gpu(client, prog.text, [key])
    h = n // 2
    counts = np.arange(n, dtype=np.uint32)
    y0, y1 = threefry2x32(key[0], key[1], counts[:h], counts[h:])
    np.testing.assert_array_equal(got[0], np.concatenate([y0, y1]))
