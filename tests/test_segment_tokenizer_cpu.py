"""Segment-consistent tokenisation and the image-code token layout."""
import torch

from mindspeed_mm_b200.data.segment_tokenizer import SegmentTokenizer, codes_from_token_ids, image_token_ids


def _sp_like(s):             # sentencepiece-like: a space is glued to the front of the text, words carry their leading space
    return [hash(w) % 1000 for w in (" " + s).replace(" ", " ▁").split(" ") if w]


def _marked(s):              # a word carries a marker only when a space really precedes it
    out, word, spaced = [], "", False
    for ch in s + " ":
        if ch == " ":
            if word:
                out.append(hash(("_" if spaced else "") + word) % 1000)
            word, spaced = "", True
        else:
            word += ch
    return out


def _plain(s):               # byte-like: what you see is what you get
    return [ord(c) for c in s]


def test_segment_style_is_probed_and_segments_match_the_full_text():
    sp = SegmentTokenizer(_sp_like, bos_id=1, eos_id=2)
    assert not sp.needs_explicit_space
    full = sp.encode("a b c")
    assert sp.encode("a b") + sp.encode_segment(" c") == full or sp.encode("a b") + sp.encode("c") == full
    mk = SegmentTokenizer(_marked, eos_id=2)
    assert mk.needs_explicit_space and mk.bos_id == 2
    assert mk.encode("a b") + mk.encode_segment(" c") == mk.encode("a b c")
    pl = SegmentTokenizer(_plain, eos_id=2)
    assert not pl.needs_explicit_space
    assert pl.encode("a b") + pl.encode_segment(" c") == pl.encode("a b c")
    assert pl.encode("x", bos=True, eos=True) == [2, ord("x"), 2]


def test_image_code_layout_round_trip():
    codes = torch.arange(6).view(2, 3)
    ids = image_token_ids(codes, code_offset=100, start_id=7, end_id=8, newline_id=9, size_token_base=50)
    assert ids == [7, 52, 53, 100, 101, 102, 9, 103, 104, 105, 9, 8]
    back = codes_from_token_ids([1, 1] + ids + [3], 100, 7, 8, 9, size_token_base=50)
    assert torch.equal(back, codes)
    assert image_token_ids(codes, 0, 7, 8, 9)[:2] == [7, 0]
