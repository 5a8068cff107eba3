"""Tokenizer and dataset tooling, one test per behaviour the reference pins (rust-nn src/tokenizer.rs:614-812,
src/data.rs:719-1368): round trips (ASCII, Unicode, raw bytes), vocabulary size, scoring modes, pre-tokenisation, offsets,
batches, persistence, specials, determinism, edge cases; CSV / JSONL parsing and type inference, dataset slicing and
tensors, synthetic generators, base64, the small JSON helpers, credentials, the dataset builder, listings. HTTP clients are
exercised against a local fake of the datasets-server response (no network)."""
import base64
import json
import os

import numpy as np
import pytest
import torch

from rust_neural_network_b200 import data as D
from rust_neural_network_b200.tokenizer import BpeTokenizer, MergeScoring, pre_tokenize

CORPUS = ("the quick brown fox jumps over the lazy dog. " * 30 + "pack my box with five dozen liquor jugs! " * 20
          + "café naïve 日本語 \U0001f600 " * 10)


@pytest.fixture(scope="module")
def tok():
    return BpeTokenizer.train(CORPUS, 400, MergeScoring.Frequency)


def test_round_trip_ascii(tok):
    s = "the quick brown fox, and the lazy dog."
    assert tok.decode(tok.encode(s)) == s


def test_round_trip_unicode(tok):
    s = "café 日本語 \U0001f600 naïve üß"
    assert tok.decode(tok.encode(s)) == s


def test_round_trip_bytes_exact(tok):
    s = "tabs\tand\nnewlines  double  spaces\r\n"
    ids = tok.encode(s)
    assert tok.decode_bytes(ids) == s.encode("utf-8")
    assert b"".join(tok.id_to_bytes(i) for i in ids) == s.encode("utf-8")


def test_vocab_size_respected(tok):
    assert 256 < tok.vocab_size <= 400 and len(tok) == tok.vocab_size and not tok.is_empty()
    small = BpeTokenizer.train("aaaa", 1000, MergeScoring.Frequency)       # a tiny corpus runs out of pairs early
    assert small.vocab_size < 1000


def test_merges_reduce_token_count(tok):
    s = "the quick brown fox jumps over the lazy dog."
    assert len(tok.encode(s)) < len(s.encode()) // 2
    assert tok.compression_ratio(s) < 0.5                                  # tokens per character, like the reference


def test_pmi_and_hybrid_scoring_work():
    for scoring in (MergeScoring.PMI, MergeScoring.Hybrid(0.3)):
        t = BpeTokenizer.train(CORPUS, 330, scoring)
        s = "pack my box with five dozen liquor jugs!"
        assert t.decode(t.encode(s)) == s and t.vocab_size > 256
    assert MergeScoring.Hybrid(0.3) != MergeScoring.Frequency


def test_pre_tokenize_partitions():
    s = "Hello, world!  It's 2024\n\nnew lineé"
    chunks = pre_tokenize(s)
    assert b"".join(c for _, c in chunks) == s.encode()                    # nothing lost, nothing duplicated
    offs = [o for o, _ in chunks]
    assert offs == sorted(offs) and offs[0] == 0


def test_pre_tokenize_word_boundaries():
    chunks = [c for _, c in pre_tokenize("hello world foo")]
    assert chunks == [b"hello", b" world", b" foo"]                        # the space travels with the word that follows


def test_encode_with_offsets_aligns(tok):
    s = "the lazy dog jumps"
    raw = s.encode()
    pieces = tok.encode_with_offsets(s)
    assert [i for i, _ in pieces] == tok.encode(s)
    covered = b"".join(raw[r.start:r.stop] for _, r in pieces)
    assert covered == raw
    for tid, r in pieces:
        assert tok.id_to_bytes(tid) == raw[r.start:r.stop]


def test_batch_encode_decode_parallel(tok):
    texts = [f"sample number {i}: the quick brown fox" for i in range(40)]
    batch = tok.encode_batch(texts, threads=4)
    assert batch == [tok.encode(t) for t in texts]
    assert tok.decode_batch(batch) == texts


def test_count_tokens_matches_encode_len(tok):
    for s in ("", "a", "the quick brown fox", CORPUS[:200]):
        assert tok.count_tokens(s) == len(tok.encode(s))


def test_save_load_round_trips(tok):
    again = BpeTokenizer.load(tok.save())
    s = "the quick café"
    assert again.vocab_size == tok.vocab_size and again.encode(s) == tok.encode(s)
    from_merges = BpeTokenizer.from_merges([(104, 101), (108, 108)])       # "he", "ll"
    assert from_merges.encode("hello") == [256, 257, 111]


def test_special_tokens(tok):
    t = BpeTokenizer.load(tok.save())
    sid = t.add_special("<|endoftext|>")
    assert sid == t.vocab_size - 1
    assert t.add_special("<|endoftext|>") == sid                            # registering twice returns the same id
    assert t.id_to_bytes(sid) == b"<|endoftext|>" and t.decode(t.encode("the dog") + [sid]) == "the dog<|endoftext|>"
    again = BpeTokenizer.load(t.save())                                     # specials survive save / load
    assert again.decode([sid]) == "<|endoftext|>"


def test_deterministic_encoding_and_training(tok):
    s = "pack my box with five dozen liquor jugs"
    assert tok.encode(s) == tok.encode(s)
    assert BpeTokenizer.train(CORPUS, 320, MergeScoring.Frequency).save() == BpeTokenizer.train(CORPUS, 320, MergeScoring.Frequency).save()


def test_empty_and_single_byte(tok):
    assert tok.encode("") == [] and tok.decode([]) == ""
    assert tok.encode("z") == [ord("z")] and tok.decode([0x41]) == "A"
    assert tok.compression_ratio("") == 0.0


# ------------------------------------------------------------------------------------------------ data
def test_csv_loading_and_type_inference(tmp_path):
    p = tmp_path / "a.csv"
    p.write_text("x,y,name\n1.5,2,alice\n-3,4e2,bob\n")
    ds = D.load_csv(str(p))
    assert ds.get_float("x").tolist() == [1.5, -3.0] and ds.get_float("y").tolist() == [2.0, 400.0]
    assert ds.get_text("name") == ["alice", "bob"] and ds.get_float("name") is None and ds.get_text("x") is None


def test_csv_quoted_fields_and_tsv(tmp_path):
    assert D.parse_csv_line('a,"b,c","d e",f') == ["a", "b,c", "d e", "f"]      # quotes toggle, the delimiter inside them is data
    p = tmp_path / "a.tsv"
    p.write_text("a\tb\n1\thello world\n")
    ds = D.load_tsv(str(p))
    assert ds.get_float("a").tolist() == [1.0] and ds.get_text("b") == ["hello world"]


def test_jsonl_loading(tmp_path):
    p = tmp_path / "a.jsonl"
    p.write_text('{"v": 1.5, "t": "one"}\n{"v": 2, "t": "two, with comma"}\n\n')
    ds = D.load_jsonl(str(p))
    assert ds.get_float("v").tolist() == [1.5, 2.0] and ds.get_text("t") == ["one", "two, with comma"]


def test_dataset_to_tensor_head_split_summary():
    ds = D.Dataset.new("mem")
    ds.add_float_column("a", [1, 2, 3, 4, 5]); ds.add_float_column("b", [10, 20, 30, 40, 50]); ds.add_text_column("t", list("vwxyz"))
    t = ds.to_tensor(["b", "a"])
    assert t.shape == (5, 2) and t[2].tolist() == [30.0, 3.0]
    assert ds.to_tensor(["t", "missing"]).abs().sum() == 0                  # text / unknown columns read as zeros
    h = ds.head(2)
    assert h.get_float("a").tolist() == [1.0, 2.0] and h.get_text("t") == ["v", "w"]
    tr, te = ds.train_test_split(0.6)                                       # the ratio is the TRAIN share, like the reference
    assert len(tr.get_float("a")) == 3 and len(te.get_float("a")) == 2 and te.get_text("t") == ["y", "z"]
    s = ds.summary()
    assert "a" in s and "f32[5]" in s and "str[5]" in s


def test_to_token_tensor_pads_and_truncates():
    tok = BpeTokenizer.from_merges([])
    ds = D.Dataset.new("m"); ds.add_text_column("t", ["abc", "abcdefgh"])
    t = ds.to_token_tensor("t", tok, 5)
    assert t.shape == (2, 5) and t[0].tolist() == [97.0, 98.0, 99.0, 0.0, 0.0] and t[1].tolist() == [97.0, 98.0, 99.0, 100.0, 101.0]


def test_synthetic_classification_and_regression():
    c = D.make_classification(90, 4, 3, seed=1)
    lab = c.get_float("label")
    assert sorted(set(lab.tolist())) == [0.0, 1.0, 2.0] and len(c.get_float("f3")) == 90
    means = [c.get_float("f0")[lab == k].mean() for k in range(3)]
    assert means[0] < means[1] < means[2]                                  # class centres are separated
    r = D.make_regression(200, 3, seed=2)
    x = np.stack([r.get_float(f"f{j}") for j in range(3)], 1)
    w, *_ = np.linalg.lstsq(x, r.get_float("target"), rcond=None)
    assert np.abs(x @ w - r.get_float("target")).max() < 0.06              # linear target + small uniform noise


def test_base64_and_json_helpers():
    for s in ("", "f", "fo", "foo", "user:keyé"):
        assert D.base64_encode(s) == base64.b64encode(s.encode()).decode()
    assert D.parse_simple_json_object('{"a": "x, y", "n": 3.5, "b": true}') == [("a", "x, y"), ("n", "3.5"), ("b", "true")]
    assert D.split_json_objects('{"a":1},{"b":{"c":2}}, {"d":"x"}') == ['{"a":1}', '{"b":{"c":2}}', '{"d":"x"}']


def test_credentials_builder_env_and_file(tmp_path, monkeypatch):
    monkeypatch.setenv("HOME", str(tmp_path))
    for k in ("HF_TOKEN", "HUGGING_FACE_HUB_TOKEN", "KAGGLE_USERNAME", "KAGGLE_KEY"):
        monkeypatch.delenv(k, raising=False)
    empty = D.Credentials.new()
    assert not empty.has_hf() and not empty.has_kaggle()
    c = D.Credentials.new().with_hf_token("hf_x").with_kaggle("me", "k")
    assert c.has_hf() and c.has_kaggle()
    c.save()
    back = D.Credentials.load()
    assert back.has_hf() and back.has_kaggle()
    monkeypatch.setenv("HF_TOKEN", "hf_env")
    assert D.Credentials.from_env().has_hf() and not D.Credentials.from_env().has_kaggle()


def test_dataset_builder_float_text_named_and_csv(tmp_path):
    b = D.DatasetBuilder.new("b").add_float_row([1.0, 2.0], 0.0).add_float_row([3.0, 4.0], 1.0)
    ds = b.build()
    assert ds.to_tensor(["f0", "f1", "label"]).tolist() == [[1.0, 2.0, 0.0], [3.0, 4.0, 1.0]]
    t = D.DatasetBuilder.new("t").add_text_row("good", "pos").add_text_row("bad", "neg").build()
    assert t.get_text("text") == ["good", "bad"] and t.get_text("label") == ["pos", "neg"]
    n = D.DatasetBuilder.new("n").add_float_column("h", [1.0, 2.0]).add_text_column("w", ["a", "b"])
    out = tmp_path / "n.csv"
    n.build_csv(str(out))
    again = D.load_csv(str(out))
    assert again.get_float("h").tolist() == [1.0, 2.0] and again.get_text("w") == ["a", "b"]


def test_format_listings_display():
    txt = D.format_listings([D.DatasetListing("org/name", "a description", 1234), D.DatasetListing("x/y", "", 0)])
    assert "org/name" in txt and "1234" in txt and "x/y" in txt
    assert D.format_listings([]) != ""


def test_huggingface_client_parses_rows_and_uses_the_cache(tmp_path, monkeypatch):
    monkeypatch.setenv("HOME", str(tmp_path))
    body = json.dumps({"rows": [{"row_idx": 0, "row": {"text": "hello", "label": 1}}, {"row_idx": 1, "row": {"text": "bye", "label": 0}}]})
    calls = []

    def fake_get(url, headers, timeout=20.0):
        calls.append((url, dict(headers)))
        return body

    monkeypatch.setattr(D, "_http_get", fake_get)
    ds = D.load_huggingface("org/set", "train", 2, D.Credentials.new().with_hf_token("hf_tok"))
    assert ds.get_text("text") == ["hello", "bye"] and ds.get_float("label").tolist() == [1.0, 0.0]
    assert "org%2Fset" in calls[0][0] or "org/set" in calls[0][0]
    assert calls[0][1].get("Authorization") == "Bearer hf_tok"
    again = D.load_huggingface("org/set", "train", 2)                       # second call is served from the cache directory
    assert len(calls) == 1 and again.get_text("text") == ["hello", "bye"]
    assert os.path.isdir(D.cache_dir())
