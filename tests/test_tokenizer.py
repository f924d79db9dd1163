"""The byte-level BPE tokenizer on a small hand-made vocabulary (no GPU)."""
import json

from sandyrt_b200.tokenizer import BPETokenizer, _byte_table


def _write(tmp_path, merges):
    table = _byte_table()
    tokens = [table[b] for b in range(256)]
    for a, b in merges:
        tokens.append(a + b)
    (tmp_path / "vocab.json").write_text(json.dumps({t: i for i, t in enumerate(tokens)}), encoding="utf-8")
    (tmp_path / "merges.txt").write_text("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges) + "\n",
                                         encoding="utf-8")
    return BPETokenizer.from_dir(str(tmp_path))


def test_byte_table_is_a_bijection_onto_printable_characters():
    t = _byte_table()
    assert len(t) == 256 and len(set(t.values())) == 256
    assert t[ord("A")] == "A" and t[ord(" ")] == chr(256 + 32) and all(not c.isspace() for c in t.values())


def test_merges_apply_by_rank_and_round_trip(tmp_path):
    sp = _byte_table()[ord(" ")]
    tok = _write(tmp_path, [("l", "l"), ("h", "e"), ("he", "ll"), (sp, "w"), ("o", "r")])
    ids = tok.encode("hello world")
    pieces = [tok.id_to_token[i] for i in ids]
    assert pieces == ["hell", "o", sp + "w", "or", "l", "d"]
    assert tok.decode(ids) == "hello world"
    for text in ("", "a", "it's 42 -- naïve\n\ttabs  ", "日本語 and emoji 🙂"):
        assert tok.decode(tok.encode(text)) == text


def test_available_needs_both_files(tmp_path):
    assert not BPETokenizer.available(str(tmp_path))
    (tmp_path / "vocab.json").write_text("{}")
    (tmp_path / "merges.txt").write_text("")
    assert not BPETokenizer.available(str(tmp_path))       # an empty vocabulary does not count
