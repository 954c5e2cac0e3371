"""TextPreprocessor, DataPipeline, the sharded DataLoader and MinHashDedup."""
import torch

from innova_b200.utils.text_pipeline import DataLoader, DataLoaderConfig, DataPipeline, MinHashDedup, TextPreprocessor
from innova_b200.utils.tokenizer import ByteTokenizer


def test_preprocessor_cleaning_rules():
    p = TextPreprocessor()
    p.set_html_stripping(True); p.set_url_removal(True); p.set_email_removal(True); p.set_lowercase(True); p.set_accent_removal(True)
    raw = "<p>Visit <a href='x'>https://example.com/a?b=1</a> or mail Jo.Doe@Mail.org &amp; call +1 415-555-2671.</p>\n\n\n\n<script>x()</script>Café   déjà  vu"
    out = p.process(raw)
    assert "<" not in out and "example.com" not in out and "mail.org" not in out and "555" not in out and "[redacted]" in out
    assert "cafe deja vu" in out and "&" in out and "  " not in out and "\n\n\n" not in out
    q = TextPreprocessor()
    assert q.process("SSN 123-45-6789, card 4111 1111 1111 1111, host 10.0.0.1") == "SSN [REDACTED], card [REDACTED], host [REDACTED]"
    q.set_pii_removal(False)
    assert "123-45-6789" in q.process("SSN 123-45-6789")
    q.set_min_length(10); q.set_max_length(12)
    assert q.process("short") == "" and q.process("a" * 30) == "a" * 12
    assert TextPreprocessor.detect_language("This is the text that it is") == "en" and TextPreprocessor.detect_language("Привет мир") == "ru"
    assert TextPreprocessor.detect_language("これは日本語です") == "ja" and TextPreprocessor.detect_language("你好世界") == "zh"
    assert TextPreprocessor.detect_language("1234 !!") == "unknown" and TextPreprocessor.detect_language("bonjour tout le monde") == "latin"


def test_deduplication_exact_and_fuzzy_and_metadata():
    p = TextPreprocessor()
    p.set_deduplication(True); p.set_fuzzy_dedup_threshold(0.8)
    a = "the quick brown fox jumps over the lazy dog near the river bank today"
    texts = [a, a, a.replace("today", "today!"), "a completely different sentence about tensors and kernels", ""]
    assert p.fuzzy_similarity(a, a) == 1.0 and p.fuzzy_similarity(a, texts[3]) < 0.1 and p.fuzzy_similarity(a, texts[2]) > 0.9
    out, langs, lens = p.process_with_metadata(texts)
    assert out == [a, texts[3]] and langs == ["en", "en"] and lens == [len(a), len(texts[3])]
    p.set_fuzzy_dedup_threshold(1.0)
    assert len(p.process_batch(texts)) == 3                         # exact repeats only


def test_pipeline_stages_and_file(tmp_path):
    pipe = DataPipeline()
    pipe.set_preprocessor(TextPreprocessor()); pipe.set_tokenizer(ByteTokenizer()); pipe.set_batch_size(2); pipe.set_seq_length(8)
    texts = ["hello world, this is document one.", "", "and here is the second document!!"]
    s1 = pipe.run_stage1(texts)
    s2 = pipe.run_stage2(s1)
    s3 = pipe.run_stage3(s2)
    assert len(s1) == 2 and [len(x) for x in s2] == [len(t) for t in s1]
    total = sum(len(x) for x in s2)
    assert len(s3) == total // 16 and all(b.shape == (2, 8) and b.dtype == torch.int64 for b in s3)
    assert torch.cat([b.reshape(-1) for b in s3]).tolist() == [t for d in s2 for t in d][: len(s3) * 16]
    pipe.add_stage("shift", lambda bs: [b + 1 for b in bs])
    out = pipe.process_texts(texts)
    assert torch.equal(out[0], s3[0] + 1) and pipe.total_processed == 3
    pipe.set_num_workers(3)
    assert [len(x) for x in pipe.run_stage2(s1)] == [len(x) for x in s2]
    f = tmp_path / "docs.txt"
    f.write_text("first paragraph of text here\n\nsecond paragraph follows it\n\n\nthird one")
    pipe.clear_pipeline()
    assert len(pipe.process_file(str(f))) == len("first paragraph of text heresecond paragraph follows itthird one") // 16 and pipe.total_processed == 3


def test_loader_shards_shuffles_and_labels(tmp_path):
    f = tmp_path / "corpus.bin"
    data = bytes(range(256)) * 8                                    # 2048 byte tokens: token value == position % 256
    f.write_bytes(data)
    seen = []
    for rank in range(2):
        dl = DataLoader(DataLoaderConfig(str(f), batch_size=2, seq_length=16, shuffle_buffer=4, num_epochs=1, seed=7, world_size=2, rank=rank))
        assert dl.num_batches() == ((2048 - 1) // 16 // 2) // 2 + (0 if rank else 0) or dl.num_batches() > 0
        starts = []
        for x, y in dl:
            assert x.shape == (2, 16) and torch.equal(y[:, :-1], x[:, 1:]) and torch.equal((x[:, 0] + 16) % 256, (y[:, -1] + 0) % 256)
            starts += x[:, 0].tolist()
        assert not dl.has_next()
        seen.append(starts)
    assert len(set(seen[0])) > 4 and seen[0] != sorted(seen[0])      # shuffled
    # the two ranks read disjoint windows of the same file (window index parity differs)
    w0 = {s // 16 % 2 for s in seen[0]}
    w1 = {s // 16 % 2 for s in seen[1]}
    assert w0 == {0} and w1 == {1}
    dl = DataLoader(DataLoaderConfig(str(f), batch_size=4, seq_length=32, num_epochs=3, shuffle_buffer=100))
    n1 = dl.num_batches()
    first = dl.next_batch()
    dl.reset()
    assert n1 == 3 * 63 // 4 and torch.equal(dl.next_batch(), first)


def test_minhash_filter_counts_and_stream():
    mh = MinHashDedup(ngram_size=4, num_hashes=32, max_capacity=100000)
    assert not mh.is_duplicate([1, 2, 3, 4])
    mh.insert([1, 2, 3, 4])
    assert mh.is_duplicate([1, 2, 3, 4]) and not mh.is_duplicate([1, 2, 3, 5]) and not mh.is_duplicate([4, 3, 2, 1])
    assert mh.total_checked == 4 and mh.duplicates_found == 1 and mh.duplicate_rate() == 0.25
    mh.clear()
    doc = list(range(100, 140))
    out = mh.filter_stream(doc + [7, 8] + doc)                      # the second copy is cut out
    assert out[:42] == doc + [7, 8] and len(out) < 42 + 8
    small = MinHashDedup(4, 8, max_capacity=64)
    for i in range(100):
        small.insert([i, i + 1, i + 2, i + 3])
    assert len(small._seen) <= 64 and not small.is_duplicate([0, 1, 2, 3]) and small.is_duplicate([99, 100, 101, 102])
