import numpy as np
import torch

from innova_b200.utils.datasets import (ChunkedDataset, ConcatDataset, FilterDataset, InMemoryDataset, MapDataset, ShuffleDataset,
                                         StreamingDataset, split_dataset)
from innova_b200.utils.tokenizer import ByteTokenizer
from innova_b200.utils.tokenizers_ext import (MultiLingualTokenizer, SentencePieceTrainer, UnigramTokenizer, WordPieceTokenizer, load_any,
                                               pretokenize_default, split_on_whitespace_and_punctuation)

CORPUS = ["the quick brown fox jumps over the lazy dog", "the dog barks and the fox runs", "quick quick brown brown foxes jumping",
          "lazy dogs are running over the quick fox"] * 5


def test_unigram_tokenizer(tmp_path):
    t = UnigramTokenizer().train(CORPUS, vocab_size=60)
    assert t.vocab_size <= 60 + 30            # single characters are always kept
    text = "the quick fox runs"
    ids, scores = t.encode_with_scores(text)
    assert t.decode(ids) == text and all(s <= 0 for s in scores)
    assert len(ids) < len(text)               # learnt multi-character pieces
    assert t.unk_id in t.encode("fox ζ")
    t.save(str(tmp_path / "u.model"))
    assert load_any(str(tmp_path / "u.model")).encode(text) == ids


def test_wordpiece_tokenizer(tmp_path):
    t = WordPieceTokenizer().train(CORPUS, vocab_size=80)
    ids = t.encode("the quick foxes", add_special=True)
    assert ids[0] == t.bos_id and ids[-1] == t.eos_id and t.decode(ids) == "the quick foxes"
    assert t.encode("zzz")[0] == t.unk_id or t.decode(t.encode("zzz")) == "zzz"
    assert any(p.startswith("##") and len(p) > 3 for p in t.vocab)
    t.save(str(tmp_path / "w.model"))
    assert load_any(str(tmp_path / "w.model")).encode("lazy dog") == t.encode("lazy dog")


def test_sentencepiece_trainer_and_pretokenisers(tmp_path):
    assert pretokenize_default("hello, world") == ["▁hello", ",", "▁world"]
    assert split_on_whitespace_and_punctuation("a-b c!") == ["a", "-", "b", "c", "!"]
    for kind in (SentencePieceTrainer.BPE, SentencePieceTrainer.UNIGRAM, SentencePieceTrainer.WORDPIECE):
        tok = SentencePieceTrainer.train(CORPUS + ["rare ☃ glyph"], str(tmp_path / f"m{kind}"), kind, vocab_size=300 if kind == 0 else 70,
                                         character_coverage=0.99)
        again = load_any(str(tmp_path / f"m{kind}.model"))
        assert again.encode("the lazy dog") == tok.encode("the lazy dog")


def test_multilingual_tokenizer(tmp_path):
    corpus = CORPUS + ["быстрая коричневая лиса", "лиса бежит быстро", "快速的棕色狐狸", "狐狸跑得很快"] * 3
    t = MultiLingualTokenizer()
    t.add_language_token("en")
    t.train(corpus, vocab_size=400)
    segs = t.split_by_language("fox лиса 狐狸")
    assert [s for s, _ in segs] == ["latin", "cyrillic", "cjk"]
    text = "the fox и лиса 和 狐狸 ☃"
    assert t.decode(t.encode(text)) == text                       # byte fallback covers everything
    ids = t.encode_with_lang_tag("привет", "ru")
    assert ids[0] >= t.bpe.vocab_size and t.decode(ids) == "привет"
    t.save(str(tmp_path / "ml.model"))
    assert load_any(str(tmp_path / "ml.model")).encode(text) == t.encode(text)


def test_dataset_combinators(tmp_path):
    text = tmp_path / "a.txt"
    text.write_text("abcdefghijklmnopqrstuvwxyz" * 8)
    ds = InMemoryDataset.from_text_file(str(text), ByteTokenizer(), seq_len=16, stride=8)
    x, y = ds.get(0)
    assert len(ds) > 10 and torch.equal(x[1:], y[:-1])
    toks = tmp_path / "t.bin"
    np.arange(1000, dtype="<i4").tofile(toks)
    dt = InMemoryDataset.from_tokenized_file(str(toks), seq_len=32)
    assert len(dt) == 31 and int(dt.get(3)[0][0]) == 96
    ch = ChunkedDataset(str(toks), chunk_size=200, overlap=40, seq_len=32)
    assert ch.num_chunks >= 6 and int(ch.get(len(ch) - 1)[1][-1]) < 1000
    xs = [int(ch.get(i)[0][0]) for i in range(len(ch))]
    assert xs == sorted(xs)
    st = StreamingDataset(str(tmp_path / "*.bin"), seq_len=32, buffer_size=8)
    seen = {int(st.get(i)[0][0]) for i in range(len(st))}
    assert len(st) == 31 and len(seen) == 31
    even = FilterDataset(dt, lambda a, b: int(a[0]) % 64 == 0)
    assert len(even) == 16
    plus = MapDataset(even, lambda a, b: (a + 1, b + 1))
    assert int(plus.get(1)[0][0]) == 65
    cat = ConcatDataset([dt, even])
    assert len(cat) == 47 and torch.equal(cat.get(31)[0], even.get(0)[0])
    sh = ShuffleDataset(dt, seed=1)
    assert sorted(int(sh.get(i)[0][0]) for i in range(len(sh))) == [32 * i for i in range(31)]
    tr, va, te = split_dataset(dt, 0.7, 0.2)
    assert len(tr) + len(va) + len(te) == 31 and len(tr) == 21 and len(va) == 6
    bx, by = next(dt.batches(4))
    assert bx.shape == (4, 32) and by.shape == (4, 32)
