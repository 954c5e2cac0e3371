"""Byte-level BPE in the Qwen layout: training, files, special tokens, chat template (CPU)."""
from innova_b200.utils.qwen_tokenizer import QwenMessage, QwenTokenizer, byte_map


def _tok():
    texts = ["the quick brown fox jumps over the lazy dog", "the dog's 3 bones, the fox's 12 hens!", "héllo wörld 你好 the the the"] * 4
    return QwenTokenizer.train(texts, vocab_size=330)


def test_byte_map_is_a_bijection_on_printable_code_points():
    m = byte_map()
    assert len(set(m.values())) == 256 and m[ord("a")] == "a" and m[ord(" ")] == chr(256 + 32) and all(not v.isspace() for v in m.values())


def test_roundtrip_merges_and_specials(tmp_path):
    t = _tok()
    assert 256 < t.vocab_size <= 333 and t.bos_id() == -1 and t.eos_id() == t.im_end_id()
    text = "the quick dog's 42 hens — héllo 你好\n\n  tabs\tand spaces  "
    ids = t.encode(text)
    assert t.decode(ids) == text and len(ids) < len(text.encode("utf-8"))          # merges compress
    assert len(t.encode("the")) == 1                                                # a frequent word became one token
    assert [len(t.encode(d)) for d in "0123456789"] == [1] * 10 and len(t.encode("12")) == 2      # digits are never merged
    s = "<|im_start|>user\nhi<|im_end|>"
    ids = t.encode(s)
    assert ids[0] == t.im_start_id() and ids[-1] == t.im_end_id() and t.is_special(ids[0]) and not t.is_special(ids[1])
    assert t.decode(ids) == "user\nhi" and t.decode(ids, skip_special=False) == s
    t.save_to_dir(str(tmp_path / "m"))
    u = QwenTokenizer.load_from_dir(str(tmp_path / "m"))
    assert u.encode(text) == t.encode(text) and u.specials == t.specials and u.vocab_size == t.vocab_size


def test_chat_template():
    t = _tok()
    msgs = [QwenMessage("system", "be brief"), QwenMessage("user", "2+2?"), QwenMessage("assistant", "4", reasoning_content="add")]
    s = t.render_chat(msgs, add_generation_prompt=True)
    assert s == ("<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\n2+2?<|im_end|>\n"
                 "<|im_start|>assistant\n<think>\nadd\n</think>\n\n4<|im_end|>\n<|im_start|>assistant\n")
    ids = t.apply_chat_template(msgs, add_generation_prompt=False)
    assert ids.count(t.im_start_id()) == 3 and ids.count(t.im_end_id()) == 3 and t.decode(ids, skip_special=False) == t.render_chat(msgs, False)
