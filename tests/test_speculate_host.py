"""Drafters of speculative decoding (host only): the plain prompt lookup with its fall-back from `ngram` tokens down to
one, and the n-gram cache (counts of continuations of the last 1..4 tokens with sample-size and share thresholds)."""
import numpy as np
import pytest

from tests import helpers


def ngram_draft_reference(seq, kmax):
    """The drafter's rule restated with dictionaries (kernels/llmrt.cu:2638-2661).  Where two continuations tie for the
    largest count the library follows its hash map's order, so this returns, per draft position, the SET of tokens that
    rule allows, following the library's own choice to continue."""
    min_n, min_pct = [2, 2, 1, 1], [66, 50, 50, 50]
    grams = {}
    for i in range(1, len(seq)):
        for n in range(1, 5):
            if i - n >= 0:
                grams.setdefault(tuple(seq[i - n:i]), {}).setdefault(seq[i], 0)
                grams[tuple(seq[i - n:i])][seq[i]] += 1

    def allowed(ctx):
        for n in range(4, 0, -1):
            if len(ctx) < n:
                continue
            part = grams.get(tuple(ctx[-n:]))
            if not part:
                continue
            best, total = max(part.values()), sum(part.values())
            if total < min_n[n - 1] or 100 * best < min_pct[n - 1] * total:
                continue
            return {t for t, c in part.items() if c == best}
        return set()

    return allowed


@pytest.fixture(scope="module")
def spec():
    helpers.build_library()
    from lazyweights_b200 import speculate
    return speculate


def test_lookup_falls_back_to_shorter_ngrams(spec):
    assert spec.lookup_draft([1, 2, 3, 9, 1, 2, 3], 3, 4) == [9, 1, 2, 3]
    assert spec.lookup_draft([1, 2, 3], 3, 4) == []
    assert spec.lookup_draft([5, 6, 7, 8, 9, 7], 3, 4) == [8, 9, 7]            # no 3- or 2-gram match: last token alone
    assert spec.lookup_draft([4, 4, 8, 1, 4, 8], 3, 2) == [1, 4]               # 2-gram (4, 8) matches, 3-gram does not
    assert spec.lookup_draft([1, 2, 1, 2], 1, 8) == [1, 2]                     # latest earlier occurrence of the last token
    assert spec.lookup_draft([3], 3, 4) == [] and spec.lookup_draft([], 3, 4) == []


def test_ngram_cache_known_answers(spec):
    d = spec.NgramCacheDrafter()
    assert d.draft([7], 4) == []                                               # fewer than two tokens: nothing
    seq = [1, 2, 3, 4, 1, 2, 3, 4, 1, 2]
    got = d.draft(seq, 6)
    assert got == [3, 4, 1, 2, 3, 4]                                           # the cycle continues, drafts feed drafts
    d2 = spec.NgramCacheDrafter()
    # the 3-gram (9, 5, 9) was followed by 6 once: one sample is enough for n = 3, and longer n-grams decide first
    assert d2.draft([9, 5, 9, 6, 9, 5, 9], 1) == [6]
    d2b = spec.NgramCacheDrafter()
    # only the 1-gram (9) has been seen before: continuations 5, 5, 6 -> 2 of 3 = 66.7 % passes the share of 66 %
    assert d2b.draft([9, 5, 7, 9, 5, 8, 9, 6, 3, 9], 1) == [5]
    d3 = spec.NgramCacheDrafter()
    # (1) -> 2 seen once: the 1-gram rule wants two samples, nothing is drafted
    assert d3.draft([1, 2, 3, 1], 3) == []
    d4 = spec.NgramCacheDrafter()
    assert d4.draft([8, 3, 8], 2) == []                                        # (8) -> 3 seen once: below the sample floor


def test_ngram_cache_follows_the_rule_on_seeded_histories(spec):
    rng = np.random.default_rng(0)
    for trial in range(40):
        vocab = int(rng.integers(3, 12))
        seq = [int(t) for t in rng.integers(0, vocab, int(rng.integers(2, 200)))]
        d = spec.NgramCacheDrafter()
        got = d.draft(seq, 8)
        allowed = ngram_draft_reference(seq, 8)
        ctx = list(seq)
        for t in got:
            assert t in allowed(ctx), (trial, ctx[-4:], t)
            ctx.append(t)
        if len(got) < 8:
            assert allowed(ctx) == set()                                       # it stopped because the rule has no candidate
        # incremental feeding gives the same drafts as feeding everything at once
        d_inc = spec.NgramCacheDrafter()
        for cut in range(1, len(seq)):
            d_inc.sync(seq[:cut])
        assert d_inc.draft(seq, 8) == got
