"""The host form of the engine's random numbers against published known answers."""
from aien_sovereign_core_mv_b200.sampling.sampler import philox4x32_10, philox_uniform


def test_philox4x32_10_known_answer_vectors():
    """The three known-answer vectors of Philox4x32-10 (ten rounds) as distributed with the
    Random123 library's kat_vectors: counter, key -> output."""
    kat = [
        ((0x00000000, 0x00000000, 0x00000000, 0x00000000), (0x00000000, 0x00000000),
         (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
        ((0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff), (0xffffffff, 0xffffffff),
         (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
        ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
         (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
    ]
    for counter, key, want in kat:
        assert philox4x32_10(counter, key) == want


def test_uniform_is_the_top_53_bits_of_the_first_two_words():
    u = philox_uniform(0, 0, 0)
    assert u == float(((0x6627e8d5 << 32) | 0xe169c58d) >> 11) / 2.0 ** 53 and 0.0 <= u < 1.0
    assert philox_uniform(1, 0, 0) != u and philox_uniform(0, 1, 0) != u and philox_uniform(0, 0, 1) != u
