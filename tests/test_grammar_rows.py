"""Masks for the verify rows of a speculative step over a constrained request (host logic of the matcher)."""
import numpy as np

from loken_b200.text.grammar import GrammarSession
from loken_b200.text.tokenizer import ByteTokenizer


def bit(mask, t):
    return (int(mask[t >> 5]) >> (t & 31)) & 1


def test_rows_follow_the_drafts_and_the_matcher_is_left_where_it_was():
    tk = ByteTokenizer(260)
    g = GrammarSession(tk, "regex", "(yes|no) [0-9]{2}")
    first = g.mask().copy()
    assert bit(first, ord("y")) and bit(first, ord("n")) and not bit(first, ord("x"))
    # every draft fits the language: one mask per row, each for its own history
    masks, d = g.rows_for_drafts([ord("y"), ord("e"), ord("s")])
    assert d == [ord("y"), ord("e"), ord("s")] and len(masks) == 4
    assert bit(masks[1], ord("e")) and not bit(masks[1], ord("o")) and bit(masks[3], ord(" "))
    assert np.array_equal(g.mask(), first)                                  # nothing was committed
    # the language refuses the second draft: rows stop there
    masks, d = g.rows_for_drafts([ord("n"), ord("x"), ord("o")])
    assert d == [ord("n")] and len(masks) == 2 and bit(masks[1], ord("o"))
    assert np.array_equal(g.mask(), first)
    masks, d = g.rows_for_drafts([ord("q")])
    assert d == [] and len(masks) == 1
    # a draft that completes the language is left to its row: nothing may follow it
    for t in b"no 4":
        assert g.accept(t)
    here = g.mask().copy()
    masks, d = g.rows_for_drafts([ord("2"), ord("7")])
    assert d == [] and len(masks) == 1 and np.array_equal(masks[0], here)
    assert np.array_equal(g.mask(), here) and not g.done()
    assert g.accept(ord("2")) and g.done()
