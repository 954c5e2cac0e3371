"""UnicodeUtil classification / UTF-8 helpers and the trainable byte-level BPE tokenizer."""
import pytest

from innova_b200.utils.tokenizers_ext import ByteLevelBPETokenizer, UnicodeUtil as U


def test_classification_and_utf8():
    assert U.is_cjk(ord("漢")) and U.is_cjk(ord("か")) and U.is_cjk(ord("한")) and not U.is_cjk(ord("a"))
    assert U.is_whitespace(0x20) and U.is_whitespace(0x3000) and U.is_whitespace(0x0A) and not U.is_whitespace(ord("x"))
    assert U.is_punctuation(ord("!")) and U.is_punctuation(ord("。")) and not U.is_punctuation(ord("+"))
    assert U.is_math_symbol(ord("+")) and U.is_math_symbol(ord("∑")) and U.is_currency(ord("€")) and not U.is_currency(ord("E"))
    assert U.is_letter(ord("é")) and U.is_digit(ord("٣")) and not U.is_digit(ord("½")) and U.is_control(0x07) and not U.is_control(0x0A)
    assert U.is_combining_mark(0x0301) and U.is_regional_indicator(0x1F1FA) and U.is_variation_selector(0xFE0F)
    assert U.is_emoji(0x1F600) and U.is_emoji_modifier(0x1F3FD) and not U.is_emoji(ord("a"))
    assert U.width(ord("a")) == 1 and U.width(ord("漢")) == 2 and U.width(0x0301) == 0 and U.width(0) == 0 and U.width(0xFF21) == 2
    assert U.compose_pair(ord("e"), 0x0301) == ord("é") and U.compose_pair(ord("x"), ord("y")) == 0
    assert U.nfkc_normalize("ﬁ①") == "fi1"
    for cp in (0x24, 0xA2, 0x20AC, 0x10348):
        enc = U.utf8_encode(cp)
        assert enc == chr(cp).encode() and U.utf8_decode(enc, 0) == (cp, len(enc))
    assert U.utf8_encode(0xD800) == "�".encode() and U.utf8_encode(-1) == "�".encode()
    assert U.utf8_to_codepoints("aé漢😀") == [0x61, 0xE9, 0x6F22, 0x1F600] and U.codepoints_to_utf8([0x61, 0x6F22]) == "a漢".encode()
    # malformed input: lone continuation, truncated sequence, overlong form, encoded surrogate
    assert U.utf8_to_codepoints(b"\x80a") == [0xFFFD, 0x61] and U.utf8_to_codepoints(b"\xe6\xbc") == [0xFFFD, 0xFFFD]
    assert U.utf8_to_codepoints(b"\xc0\xaf") == [0xFFFD, 0xFFFD] and U.utf8_to_codepoints(b"\xed\xa0\x80")[0] == 0xFFFD


def test_pretokenize_and_language():
    assert U.pretokenize("Hello, wörld 42!") == ["Hello", ",", "wörld", "42", "!"]
    assert U.pretokenize("漢字abc") == ["漢", "字", "abc"] and U.pretokenize("éx") == ["éx"]
    assert U.pretokenize("hi 👍🏽 🇺🇸!") == ["hi", "👍🏽", "🇺🇸", "!"] and U.pretokenize("👨‍👩‍👧 ok") == ["👨‍👩‍👧", "ok"]
    assert U.split_on_whitespace(" a\tb\n c ") == ["a", "b", "c"] and U.pretokenize("   ") == []
    assert U.detect_language("привет мир") == "ru" and U.detect_language("こんにちは") == "ja" and U.detect_language("hello") == "en"
    assert U.detect_language("漢字 and a bit") == "en" and U.detect_language("123 !!") == "und"


def test_byte_level_bpe_trains_and_round_trips(tmp_path):
    tok = ByteLevelBPETokenizer()
    assert tok.vocab_size() == 261 and (tok.unk_id, tok.bos_id, tok.eos_id) == (0, 3, 4) and len(set(tok.alphabet)) == 256
    assert tok.alphabet[ord("A")] == "A" and tok.alphabet[0x20] == "Ġ" and all(c.isprintable() for c in tok.alphabet)
    corpus = ["the cat sat on the mat", "the dog sat on the log", "the the the cat", "naïve café 漢字 😀"] * 5
    tok.train(corpus, vocab_size=300)
    assert 261 < tok.vocab_size() <= 300 and tok.id_to_token[261] in ("Ġt", "th", "he", "Ġth") and "Ġthe" in tok.token_to_id
    ids = tok.encode("the cat sat")
    assert len(ids) < len("the cat sat".encode()) and tok.decode(ids) == "the cat sat"
    for text in ("", "  leading and trailing  ", "naïve café 漢字 😀\n\tnew", "unseen: zyxw 9876 #$%"):
        assert tok.decode(tok.encode(text)) == text
    wrapped = tok.encode("the", add_special=True)
    assert wrapped[0] == 3 and wrapped[-1] == 4 and tok.decode(wrapped) == "the"
    # merges are applied in training order: re-encoding from raw bytes gives the same ids as the cached path
    assert tok.bpe_merge_tokens(tok.byte_encode(" the")) == tok.encode(" the") == [tok.token_to_id["Ġthe"]]
    path = str(tmp_path / "bbpe.json")
    tok.save(path)
    other = ByteLevelBPETokenizer()
    other.load(path)
    assert other.id_to_token == tok.id_to_token and other.encode("the dog sat on the mat") == tok.encode("the dog sat on the mat")
    (tmp_path / "bad.json").write_text('{"type": "byte_level_bpe", "merges": [[5, 99999]]}')
    with pytest.raises(ValueError):
        other.load(str(tmp_path / "bad.json"))
    (tmp_path / "bad2.json").write_text('{"type": "other"}')
    with pytest.raises(ValueError):
        other.load(str(tmp_path / "bad2.json"))
    small = ByteLevelBPETokenizer()
    small.train(["ab"], vocab_size=400)                     # no pair reaches the minimum frequency: nothing is merged
    assert small.vocab_size() == 261
