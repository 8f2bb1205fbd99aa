"""Host Philox-4x32-10: published known-answer vectors of the algorithm, the stream layout of
the reference generator (ferrotorch-gpu/src/rng.rs:2651-2950), the per-device manager."""
import numpy as np
import pytest

from ferrotorch_b200.utils import philox as P


def test_known_answers():
    # Random123's kat_vectors for philox4x32-10: (counter words, key words) -> output words
    z = P.philox_4x32_10(0, 0)
    assert [hex(v) for v in z] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    f = P.philox_4x32_10(0xFFFFFFFFFFFFFFFF, 0xFFFFFFFFFFFFFFFF, 0xFFFFFFFFFFFFFFFF)
    assert [hex(v) for v in f] == ["0x408f276d", "0x41c83b0e", "0xa20bc7c6", "0x6d5451fd"]
    pi = P.philox_4x32_10(0x85A308D3243F6A88, 0x299F31D0A4093822, 0x0370734413198A2E)
    assert [hex(v) for v in pi] == ["0xd16cfe09", "0x94fdcceb", "0x5001e420", "0x24126ea1"]


def test_stream_layout_and_state():
    g = P.PhiloxGenerator(42)
    first = g.next_u32()
    assert (g.counter, g.offset) == (0, 1)
    for _ in range(3):
        g.next_u32()
    assert (g.counter, g.offset) == (1, 0)
    g.set_seed(42)
    assert g.next_u32() == first and first == int(P.philox_4x32_10(0, 42)[0])
    # words drawn one at a time equal words drawn in bulk, across counter boundaries
    a = P.PhiloxGenerator(7)
    one = [a.next_u32() for _ in range(11)]
    b = P.PhiloxGenerator(7)
    assert list(b.words(3)) + list(b.words(6)) + list(b.words(2)) == one and b.get_state() == a.get_state()
    # save in the middle of a counter, restore, continue
    st = a.get_state()
    assert st.offset == 3
    nxt = [a.next_u32() for _ in range(5)]
    c = P.PhiloxGenerator(0)
    c.set_state(st)
    assert [c.next_u32() for _ in range(5)] == nxt
    c.advance(10)
    assert c.offset == 0 and c.counter == a.get_state().counter + 10
    with pytest.raises(ValueError):
        P.PhiloxState.from_parts(0, 0, 4)


def test_uniform_and_normal_statistics():
    g = P.PhiloxGenerator(123)
    u = g.generate_uniform(200000)
    assert u.dtype == np.float32 and 0 <= u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 5e-3
    assert abs(u.var() - 1 / 12) < 2e-3
    n = g.generate_normal(200001)
    assert n.shape == (200001,) and abs(n.mean()) < 1e-2 and abs(n.std() - 1) < 1e-2
    # same pairs as the scalar definition
    h = P.PhiloxGenerator(5)
    u1, u2 = h.next_f32(), h.next_f32()
    r, th = np.sqrt(-2 * np.log(np.float32(u1))), 2 * np.pi * u2
    h.set_seed(5)
    np.testing.assert_allclose(h.generate_normal(2), [r * np.cos(th), r * np.sin(th)], rtol=1e-5)


def test_manager_fork_join():
    m = P.cuda_rng_manager()
    m.manual_seed_all(42)
    assert m.get_rng_state(0).seed == 42 and m.get_rng_state(3).seed == 42
    m.manual_seed(1, 12345)
    assert m.get_rng_state(1) == P.PhiloxState(0, 12345, 0)
    saved = P.fork_rng([0, 1])
    a = m.generator(0).generate_uniform(5)
    m.generator(1).next_u32()
    P.join_rng([0, 1], saved)
    np.testing.assert_array_equal(m.generator(0).generate_uniform(5), a)
    assert m.get_rng_state(1).offset == 0
    with pytest.raises(ValueError):
        P.join_rng([0], saved)


def test_native_word_stream_equals_numpy_rounds():
    if P._native_fill() is None:
        pytest.skip("host library not built")
    for seed, skip, n in ((0, 0, 17), (42, 3, 1), (2 ** 63 + 5, 6, 1001), (7, 2, 2)):
        g = P.PhiloxGenerator(seed)
        g.words(skip)
        st = g.get_state()
        got = g.words(n)
        blocks = (st.offset + n + 3) // 4
        ref = P.philox_4x32_10(np.arange(blocks, dtype=np.uint64) + np.uint64(st.counter), seed).reshape(-1)[st.offset:st.offset + n]
        assert np.array_equal(got, ref) and g.get_state() == P.PhiloxState(st.counter + (st.offset + n) // 4, seed, (st.offset + n) % 4)
