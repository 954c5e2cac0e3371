"""MmapDataLoader (windowed tokenisation, exact n-gram de-duplication, shuffled sequence draws) and StreamingDataLoader."""
import numpy as np
import torch

from innova_b200.utils.text_pipeline import MmapDataLoader, MmapDataLoaderConfig, StreamingDataLoader


class ByteTok:
    def encode(self, text):
        return list(text.encode("utf-8"))


class WordTok:
    def __init__(self):
        self.ids = {}

    def encode(self, text):
        return [self.ids.setdefault(w, len(self.ids) + 1) for w in text.split()]


def test_sequential_batches_cover_the_file_in_order(tmp_path):
    text = "".join(f"line {i:05d} é\n" for i in range(400))
    p = tmp_path / "c.txt"
    p.write_text(text, encoding="utf-8")
    raw = list(text.encode("utf-8"))
    cfg = MmapDataLoaderConfig(batch_size=2, seq_length=16, shuffle_buffer=0, mmap_window=300, dedup_enabled=False)
    with MmapDataLoader(str(p), ByteTok(), cfg) as dl:
        got, pairs = [], 0
        while dl.has_next():
            b = dl.next_batch_with_labels()
            if b is None:
                break
            ids, lab = b
            assert ids.shape == lab.shape == (2, 16) and torch.equal(ids.flatten()[1:], lab.flatten()[:-1])
            got.extend(ids.flatten().tolist())
            pairs += 1
        assert got == raw[: len(got)] and len(raw) - len(got) <= 2 * 16 and dl.num_batches() - pairs in (0, 1) and dl.total_tokens == len(raw)
        dl.reset()
        assert torch.equal(dl.next_batch(), torch.tensor(raw[:32]).view(2, 16))
    # windows never split a UTF-8 sequence: no replacement characters appear with a tiny window
    with MmapDataLoader(str(p), ByteTok(), MmapDataLoaderConfig(1, 8, 0, 7, False)) as dl2:
        seen = []
        while (b := dl2.next_batch()) is not None:
            seen.extend(b.flatten().tolist())
        assert bytes(seen).decode("utf-8", "ignore") == text[: len(bytes(seen).decode("utf-8", "ignore"))] and 0xEF not in seen
    empty = tmp_path / "e.txt"
    empty.write_bytes(b"")
    e = MmapDataLoader(str(empty), ByteTok(), cfg)
    assert not e.has_next() and e.next_batch() is None
    e.close()


def test_ngram_dedup_drops_repeats_within_and_across_windows(tmp_path):
    unique = [f"w{i}" for i in range(600)]
    para = " ".join(unique[:50])
    text = " ".join(unique[:300]) + "\n" + para + "\n" + " ".join(unique[300:]) + "\n" + para + "\n"
    p = tmp_path / "d.txt"
    p.write_text(text)
    cfg = MmapDataLoaderConfig(batch_size=1, seq_length=32, shuffle_buffer=0, mmap_window=900, dedup_enabled=True, ngram_size=4)
    tok = WordTok()
    with MmapDataLoader(str(p), tok, cfg) as dl:
        out = []
        while (b := dl.next_batch()) is not None:
            out.extend(b.flatten().tolist())
        total, dropped = dl.total_tokens, dl.tokens_dropped
    assert total + dropped == 700 and 90 <= dropped <= 100                  # both repeated paragraphs go, bar the last n-1 tokens of each
    assert len(out) - len(set(out)) <= 2 * 3                               # only the last n-1 tokens of a repeated paragraph can be served again
    plain = MmapDataLoader(str(p), WordTok(), MmapDataLoaderConfig(1, 32, 0, 900, False))
    while plain.next_batch() is not None:
        pass
    assert plain.total_tokens == 700 and plain.tokens_dropped == 0
    plain.close()


def test_shuffled_draws_are_whole_sequences_and_seeded(tmp_path):
    text = " ".join(str(i) for i in range(4000)) + "\n"
    p = tmp_path / "s.txt"
    p.write_text(text)

    class NumTok:
        def encode(self, t):
            return [int(w) for w in t.split()]

    def run(seed):
        cfg = MmapDataLoaderConfig(batch_size=2, seq_length=10, shuffle_buffer=400, mmap_window=2000, dedup_enabled=False, seed=seed)
        with MmapDataLoader(str(p), NumTok(), cfg) as dl:
            rows = []
            while (b := dl.next_batch_with_labels()) is not None:
                ids, lab = b
                assert torch.equal(lab, ids + 1)                            # consecutive numbers: labels are the next token of the same row
                rows.extend(ids.tolist())
            return rows

    a, b, c = run(1), run(1), run(2)
    assert a == b and a != c and all(r == list(range(r[0], r[0] + 10)) for r in a)
    starts = [r[0] for r in a]
    assert len(set(starts)) == len(starts) and starts != sorted(starts) and len(a) >= 380


def test_streaming_loader(tmp_path):
    text = "".join(f"row {i} ü\n" for i in range(3000))
    p = tmp_path / "t.txt"
    p.write_text(text, encoding="utf-8")
    raw = list(text.encode("utf-8"))
    sl = StreamingDataLoader(ByteTok(), str(p), batch_size=4, seq_length=64, chunk_bytes=1000)
    assert sl.batch_size() == 4 and sl.seq_length() == 64
    got = []
    while (b := sl.next_batch()) is not None:
        ids, lab = b
        assert ids.shape == (4, 64) and torch.equal(ids.flatten()[1:], lab.flatten()[:-1])
        got.extend(ids.flatten().tolist())
    assert got == raw[: len(got)] and len(raw) - len(got) <= 4 * 64 and sl.num_batches() == len(got) // 256
    sl.reset()
    assert torch.equal(sl.next_batch()[0].flatten(), torch.tensor(raw[:256]))
    sl.close()
