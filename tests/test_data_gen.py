"""Synthetic tasks, curriculum promotion, tokenizer evaluation and Parquet reading (CPU)."""
import torch

from innova_b200.utils.data_gen import (CurriculumGenerator, CurriculumStage, DataGenerator, ParquetReader, TokenizerEvaluator)
from innova_b200.utils.tokenizer import ByteTokenizer


def test_generator_tasks_are_deterministic_and_well_formed():
    g, h = DataGenerator(7), DataGenerator(7)
    assert g.random_string(12) == h.random_string(12) and g.random_sentence(5) == h.random_sentence(5)
    assert len(g.random_sequence(9, 10)) == 9 and all(0 <= v < 10 for v in g.random_sequence(50, 10))
    for line in g.arithmetic_task(20):
        lhs, rhs = line.split(" = ")
        a, op, b = lhs.split()
        assert DataGenerator.compute_arithmetic(int(a), int(b), op) == int(rhs)
    assert DataGenerator.compute_arithmetic(7, 0, "/") == 0 and g.format_arithmetic_problem(6, 3, "/") == "6 / 3 = 2"
    for line in g.copy_task(5, 6):
        a, b = line[len("copy: "):].split(" -> ")
        assert a == b and len(a) == 6
    for line in g.reverse_task(5, 6):
        a, b = line[len("reverse: "):].split(" -> ")
        assert a[::-1] == b
    s = g.ngram_task(3, order=2, length=40)
    assert all(len(x) == 40 for x in s)
    assert g.passes_task_weight(1.0) and not g.passes_task_weight(0.0)


def test_curriculum_promotes_on_sustained_accuracy():
    c = CurriculumGenerator.default(seed=1)
    seen = []
    c.set_progress_fn(lambda name, d, acc: seen.append((name, d)))
    assert c.current_stage_name() == "copy" and c.current_difficulty() == 1
    b = c.generate_next_batch(4)
    assert len(b) == 4 and b[0].startswith("copy")
    c.report_accuracy(0.5)
    assert c.current_stage_name() == "copy" and not c.should_promote()
    for _ in range(3):
        c.generate_next_batch(2)
        c.report_accuracy(0.95)
    assert c.current_stage_name() == "reverse" and seen[0] == ("copy", 1)
    for stage in ("reverse", "ngram", "arithmetic"):
        for _ in range(3):
            c.generate_next_batch(2)
            c.report_accuracy(1.0)
    assert c.is_complete() and c.current_stage_name() == "arithmetic"
    c2 = CurriculumGenerator()
    c2.add_stage(CurriculumStage("hard", 5, lambda n: ["h"] * n))
    c2.add_stage(CurriculumStage("easy", 1, lambda n: ["e"] * n))
    assert c2.generate_next_batch(2) == ["e", "e"]            # stages are ordered by difficulty


def test_tokenizer_evaluator_on_the_byte_tokenizer():
    ev = TokenizerEvaluator(ByteTokenizer())
    text = "hello wörld"
    assert ev.compression_ratio(text) == 1.0 and ev.re_encoding_accuracy(text) == 1.0 and ev.reconstruction_fidelity(text) == 1.0
    assert ev.vocabulary_coverage(text) == 1.0 and ev.average_token_length(text) < 1.0
    assert TokenizerEvaluator.character_error_rate("kitten", "sitting") == 3 / 6
    rep = ev.evaluate(["abc", "", "de fg"])
    assert rep.documents == 2 and 0 < rep.vocabulary_utilization < 0.1 and "round-trip 100.0%" in ev.report_string(rep)


def test_parquet_reader(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq
    p = str(tmp_path / "shard.parquet")
    pq.write_table(pa.table({"text": ["abc", "de", None, "fghij"], "ids": [[1, 2], [3], [], [4, 5, 6]]}), p, row_group_size=2)
    r = ParquetReader("text", ByteTokenizer(), eos_id=0)
    assert not r.open(str(tmp_path / "missing.parquet")) and r.open(p) and r.shard.num_rows == 4
    a = r.next_batch(5)
    b = r.next_batch(100)
    want = list(b"abc") + [0] + list(b"de") + [0] + list(b"fghij") + [0]
    assert a.tolist() + b.tolist() == want and r.next_batch(4).numel() == 0
    assert r.total_tokens == len(want) and r.rows_read == 4
    r.reset()
    assert r.next_batch(3).tolist() == want[:3]
    r2 = ParquetReader("ids")
    assert r2.open(p) and r2.next_batch(10).tolist() == [1, 2, 3, 4, 5, 6]
    assert not ParquetReader("nope").open(p)
    r.reset()
    pairs = list(r.batches(1, 4))
    assert len(pairs) == 3 and torch.equal(pairs[0][1], torch.tensor([want[1:5]])) and torch.equal(pairs[1][0], torch.tensor([want[4:8]]))
    r.close()
