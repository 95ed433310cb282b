"""The attention part's launch plan for decoding requests (no GPU needed)."""

from mini_llm_stack_b200.parts.attention import context_splits


def test_equal_requests_fill_one_round_of_ctas():
    # eight requests of 8,192 keys and eight kv heads: 64 pairs, 296 CTAs at a time
    assert context_splits([128] * 8, 8, 296, 8) == 4
    # 512 pairs are more than a round already
    assert context_splits([128] * 64, 8, 296, 8) == 1
    # a short context is not cut below 256 keys a stretch
    assert context_splits([16], 8, 296, 8) <= 4
    assert context_splits([3], 8, 296, 8) == 1


def test_one_long_request_among_short_ones_is_cut():
    """The stretches follow the longest request; the short ones fill one stretch each,
    so the long request's tiles are what the cost counts."""
    alone = context_splits([128], 8, 296, 8)
    mixed = context_splits([128] + [4] * 63, 8, 296, 8)
    assert alone > 1 and mixed > 1
    per = -(-128 // mixed)
    busy = (-(-128 // per) + 63 * 1) * 8
    assert busy <= 2 * 296                      # the CTAs with tiles fit two rounds
    assert per <= 32                            # no CTA walks a quarter of the long context


def test_a_forced_number_of_splits(monkeypatch):
    monkeypatch.setenv("MLS_B200_SPLITS", "5")
    assert context_splits([128] * 8, 8, 296, 8) == 5
    assert context_splits([3], 8, 296, 8) == 3      # never more stretches than tiles
