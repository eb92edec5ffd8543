"""stablehlo.rng_bit_generator: Philox-4x32-10 keyed and counted by the state. The oracle's generator is pinned to the
three known-answer vectors published with the algorithm (Random123, kat_vectors: philox4x32 with ten rounds), the GPU
path is held bit-exact to the oracle. What the reference's own test asks (tests/test_ops.py:337-363: shape and type of
the output, a state that changes, the same state giving the same output and next state) is asserted as well, and the
counter advances by one per 16 bytes of output as in src/pjrt_plugin/ops/control_flow.cc:2346-2356."""
import numpy as np
import pytest

import b200
from b200.shlo.builder import Builder
from oracle import interp

KAT = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
       ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
       ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]


@pytest.mark.parametrize("ctr,key,want", KAT)
def test_philox_known_answers(ctr, key, want):
    got = interp.Interp.philox4x32_10([np.array([c], np.uint64) for c in ctr], key)
    assert tuple(int(v[0]) for v in got) == want


def _program(state_shape, state_dt, shape, dt):
    b = Builder()
    return b.module(b.rng_bit_generator(b.arg(state_shape, state_dt), shape, dt))


def test_oracle_stream_and_state():
    """The bytes of the output are the head of one stream: a shorter request is a prefix, the known-answer block is its
    first 16 bytes, and a second call with the returned state continues where a whole number of blocks ended."""
    state = np.array([0, 0], np.uint64)
    s1, a = interp.run_text(_program((2,), "ui64", (8,), "ui32"), [state])
    assert a.dtype == np.uint32 and a.shape == (8,)
    assert tuple(int(v) for v in a[:4]) == KAT[0][2]
    assert s1.dtype == np.uint64 and list(s1) == [0, 2]
    _, short = interp.run_text(_program((2,), "ui64", (5,), "ui8"), [state])
    np.testing.assert_array_equal(short, a.view(np.uint8)[:5])
    _, wide = interp.run_text(_program((2,), "ui64", (3,), "ui64"), [state])
    np.testing.assert_array_equal(wide.view(np.uint32), a[:6])
    s2, rest = interp.run_text(_program((2,), "ui64", (4,), "ui32"), [s1])
    _, both = interp.run_text(_program((2,), "ui64", (12,), "ui32"), [state])
    np.testing.assert_array_equal(np.concatenate([a, rest]), both)
    assert list(s2) == [0, 3]
    # the reference's own case: four 32-bit state words, eight words out
    st32 = np.array([0, 0, 0, 42], np.uint32)
    n1, o1 = interp.run_text(_program((4,), "ui32", (8,), "ui32"), [st32])
    n2, o2 = interp.run_text(_program((4,), "ui32", (8,), "ui32"), [st32])
    assert n1.shape == st32.shape and not np.array_equal(n1, st32)
    np.testing.assert_array_equal(o1, o2)
    np.testing.assert_array_equal(n1, n2)
    # a counter that wraps carries into the upper half of a 128-bit counter
    big = np.array([7, (1 << 64) - 1, 5], np.uint64)
    n3, _ = interp.run_text(_program((3,), "ui64", (16,), "ui32"), [big])
    assert list(n3) == [7, 3, 6]


def test_rng_plan_is_one_kernel():
    plan, _ = b200.compile_to_plan(_program((2,), "ui64", (1000, 3), "ui16"), validate=True)
    assert plan.count("rng_bits") == 1, plan
    with pytest.raises(Exception, match="16 or 24 bytes"):
        b200.compile_to_plan(_program((5,), "ui32", (8,), "ui32"))


GPU_CASES = [((2,), "ui64", (8,), "ui32"), ((4,), "ui32", (8,), "ui32"), ((2,), "ui64", (5,), "ui8"), ((2,), "ui64", (3, 7), "ui16"),
             ((2,), "ui64", (1025, 3), "ui64"), ((3,), "ui64", (1 << 20,), "ui32"), ((2,), "ui64", (0,), "ui32"), ((2,), "ui64", (33,), "i32")]


@pytest.mark.gpu
@pytest.mark.parametrize("sshape,sdt,shape,dt", GPU_CASES)
def test_rng_bit_generator_on_the_gpu(client, sshape, sdt, shape, dt):
    from util import run_gpu
    text = _program(sshape, sdt, shape, dt)
    rng = np.random.default_rng(9)
    for state in (np.zeros(sshape, np.uint64 if sdt == "ui64" else np.uint32),
                  rng.integers(0, 1 << 32, sshape).astype(np.uint64 if sdt == "ui64" else np.uint32) * (0xFFFFFFFF if sdt == "ui64" else 1)):
        if sdt == "ui64":
            state = state.copy()
            state[1] = (1 << 64) - 3 if state[0] else 0                 # the second state crosses a counter wrap
        got, _ = run_gpu(client, text, [state], dtypes=[sdt])
        want = interp.run_text(text, [state])
        np.testing.assert_array_equal(got[0], want[0])
        np.testing.assert_array_equal(got[1], want[1])


@pytest.mark.gpu
def test_rng_bits_look_uniform(client):
    """A coarse sanity check of the stream as a whole: every bit position of 2^20 words is set about half the time."""
    from util import run_gpu
    got, _ = run_gpu(client, _program((2,), "ui64", (1 << 20,), "ui32"), [np.array([1234, 0], np.uint64)], dtypes=["ui64"])
    bits = (got[1][:, None] >> np.arange(32, dtype=np.uint32)[None]) & 1
    assert np.all(np.abs(bits.mean(0) - 0.5) < 0.005)
