"""CPU tests of the I/O and tooling layer: tokenizer, dataset parsers, tiered store, REPL, dashboards,
and the BLAS / SIMD / fused / compiled / GPU-backend surfaces on their CPU paths."""
import io
import math
import os
import struct

import numpy as np
import pytest
import torch

from rust_neural_network_b200 import blas, compiled, data as D, fused, gpu, gpu_kernels, gui, interactive, nn, offload, simd
from rust_neural_network_b200.tokenizer import BpeTokenizer, MergeScoring, pre_tokenize


# ------------------------------------------------------------------ tokenizer
def test_pretokenizer_chunks():
    chunks = pre_tokenize("hello  world42!é x")
    assert [c for _, c in chunks] == [b"hello", b"  world", b"42", b"!", "é".encode(), b" x"]
    assert [s for s, _ in chunks] == [0, 5, 12, 14, 15, 17]
    assert pre_tokenize("") == []


@pytest.mark.parametrize("scoring", [MergeScoring.Frequency, MergeScoring.PMI, MergeScoring.Hybrid(0.5)])
def test_bpe_round_trip_and_compression(scoring):
    corpus = "hello world hello there world hello " * 20 + "the quick brown fox jumps over the lazy dog. " * 10
    tok = BpeTokenizer.train(corpus, 300, scoring)
    assert 256 < tok.vocab_size <= 300 and len(tok.merges) == tok.vocab_size - 256
    for text in ("hello world hello there", "unseen wörds ünd 123 numbers\n\ttabs", ""):
        ids = tok.encode(text)
        assert tok.decode(ids) == text and tok.count_tokens(text) == len(ids)
    assert tok.compression_ratio("hello world hello world") < 1.0
    assert all(0 <= i < tok.vocab_size for i in tok.encode(corpus))


def test_bpe_merge_order_and_offsets():
    tok = BpeTokenizer.train("aaabdaaabac", 259, MergeScoring.Frequency)
    # 'aa' is the most frequent pair, then ('aa','a') vs ('a','b'): counts decide, ties to the smaller pair
    assert tok.merges[0] == (97, 97)
    assert tok.id_to_bytes(256) == b"aa" and tok.id_to_bytes(97) == b"a" and tok.id_to_bytes(10 ** 6) == b""
    text = "aaab aab"
    offs = tok.encode_with_offsets(text)
    assert "".join(text.encode()[r.start:r.stop].decode() for _, r in offs) == text
    assert [i for i, _ in offs] == tok.encode(text)
    # the lowest-rank merge is applied first: with merges [(a,b)->256, (b,c)->257] "abc" -> [256, c]
    t2 = BpeTokenizer.from_merges([(97, 98), (98, 99)])
    assert t2.encode("abc") == [256, 99] and t2.encode("bc") == [257] and t2.len() == 258 and not t2.is_empty()
    assert BpeTokenizer.from_merges([]).is_empty()


def test_bpe_specials_save_load_batch():
    tok = BpeTokenizer.train("low lower lowest newer newest " * 30, 280, MergeScoring.Hybrid(0.3))
    eos = tok.add_special("<|eos|>")
    assert eos == tok.vocab_size - 1 and tok.add_special("<|eos|>") == eos and tok.decode([eos]) == "<|eos|>"
    nl = tok.add_special("a\nb")
    saved = tok.save()
    assert saved.startswith("# scoring=Hybrid") and "# specials" in saved and "a\\nb" in saved
    back = BpeTokenizer.load(saved)
    assert back.merges == tok.merges and back.vocab_size == tok.vocab_size and back.decode([nl]) == "a\nb"
    assert back.scoring.kind == "Hybrid"
    texts = ["lowest newer", "", "new low", "x" * 1000]
    assert tok.encode_batch(texts, threads=3) == [tok.encode(t) for t in texts]
    assert tok.decode_batch(tok.encode_batch(texts)) == texts
    assert tok.decode_bytes(tok.encode("héllo")) == "héllo".encode()
    with pytest.raises(ValueError):
        BpeTokenizer.train("abc", 100)


def test_bpe_long_chunk_is_fast():
    tok = BpeTokenizer.train("ab" * 200 + " abab " * 50, 270)
    text = "ab" * 50000                      # one 100k-byte chunk: the heap-based encoder stays near-linear
    ids = tok.encode(text)
    assert tok.decode(ids) == text and len(ids) < 30000


# ------------------------------------------------------------------ data
def test_csv_jsonl_parsing(tmp_path):
    p = tmp_path / "a.csv"
    p.write_text('name,age,score\n"Smith, J",30,1.5\nBob,25,-2e1\n\nEve,41,inf\n')
    ds = D.load_csv(str(p))
    assert ds.num_rows == 3 and ds.get_text("name") == ["Smith, J", "Bob", "Eve"]
    assert ds.get_float("age").tolist() == [30.0, 25.0, 41.0] and ds.get_float("score")[1] == -20.0 and math.isinf(ds.get_float("score")[2])
    assert ds.get_float("name") is None and ds.get_text("age") is None
    t = tmp_path / "a.tsv"
    t.write_text("x\ty\n1\ta\n2\tb\n")
    ts = D.load_tsv(str(t))
    assert ts.get_float("x").tolist() == [1.0, 2.0] and ts.get_text("y") == ["a", "b"]
    j = tmp_path / "a.jsonl"
    j.write_text('{"text": "hi, there", "label": 1}\n{"text": "yo \\"q\\"", "label": 0}\n')
    js = D.load_jsonl(str(j))
    assert js.get_text("text")[0] == "hi, there" and js.get_float("label").tolist() == [1.0, 0.0]
    with pytest.raises(D.DataError):
        D.load_csv(str(tmp_path / "missing.csv"))
    with pytest.raises(D.DataError):
        D.parse_delimited("\n\n", ",")
    assert D.parse_csv_line('a,"b,c",d') == ["a", "b,c", "d"]
    assert dict(D.parse_simple_json_object('{"name": "test", "value": 42}')) == {"name": "test", "value": "42"}
    assert D.split_json_objects('[{"a":1},{"b":{"c":2}}]') == ['{"a":1}', '{"b":{"c":2}}']
    assert D.base64_encode("user:key") == "dXNlcjprZXk="


def test_dataset_ops_and_synthetic():
    ds = D.make_classification(100, 4, 3, seed=0)
    assert ds.num_rows == 100 and len(ds.columns) == 5 and set(ds.get_float("label").tolist()) == {0.0, 1.0, 2.0}
    x = ds.to_tensor(["f0", "f1", "missing"])
    assert tuple(x.shape) == (100, 3) and float(x[:, 2].abs().sum()) == 0.0
    m0 = ds.get_float("f0")[ds.get_float("label") == 0].mean()
    m2 = ds.get_float("f0")[ds.get_float("label") == 2].mean()
    assert abs(m0 - 0.0) < 0.1 and abs(m2 - 1.6) < 0.1
    tr, te = ds.train_test_split(0.8)
    assert tr.num_rows == 80 and te.num_rows == 20 and "(train)" in tr.source
    assert ds.head(7).num_rows == 7 and ds.head(1000).num_rows == 100
    s = ds.summary()
    assert "rows: 100" in s and "f0: f32[100]" in s and "synthetic" in s
    reg = D.make_regression(50, 3, seed=1)
    assert reg.get_float("target").shape == (50,)
    X = reg.to_tensor(["f0", "f1", "f2"]).double()
    w = torch.linalg.lstsq(X, torch.from_numpy(reg.get_float("target")).double()[:, None]).solution
    assert float((X @ w - torch.from_numpy(reg.get_float("target")).double()[:, None]).abs().max()) < 0.06
    txt = D.Dataset("t")
    txt.add_text_column("text", ["hello world", "hello"])
    tok = BpeTokenizer.train("hello world " * 10, 260)
    tt = txt.to_token_tensor("text", tok, 6)
    assert tuple(tt.shape) == (2, 6) and tt.dtype == torch.float32 and float(tt[1, -1]) == 0.0


def test_builder_credentials_listings(tmp_path, monkeypatch):
    b = D.DatasetBuilder.new("mine").add_float_row([1.0, 2.0], 0.0).add_float_row([3.0, 4.5], 1.0)
    ds = b.build()
    assert ds.num_rows == 2 and ds.get_float("f1").tolist() == [2.0, 4.5] and ds.get_float("label").tolist() == [0.0, 1.0]
    t = D.DatasetBuilder("txt").add_text_row("good", "pos").add_text_row("bad", "neg").build()
    assert t.get_text("text") == ["good", "bad"] and t.get_text("label") == ["pos", "neg"]
    p = tmp_path / "out.csv"
    D.DatasetBuilder("c").add_float_column("x", [1.0, 2.5]).add_text_column("s", ["a", "b"]).build_csv(str(p))
    back = D.load_csv(str(p))
    assert back.get_float("x").tolist() == [1.0, 2.5] and back.get_text("s") == ["a", "b"]
    monkeypatch.setenv("HOME", str(tmp_path))
    for k in ("HF_TOKEN", "HUGGING_FACE_HUB_TOKEN", "KAGGLE_USERNAME", "KAGGLE_KEY"):
        monkeypatch.delenv(k, raising=False)
    c = D.Credentials.new()
    assert not c.has_hf() and not c.has_kaggle()
    c = c.with_hf_token("hf_x").with_kaggle("u", "k")
    assert c.has_hf() and c.has_kaggle()
    c.save()
    assert oct(os.stat(tmp_path / ".rust-nn" / "credentials.toml").st_mode & 0o777) == "0o600"
    l = D.Credentials.load()
    assert (l.hf_token, l.kaggle_username, l.kaggle_key) == ("hf_x", "u", "k")
    monkeypatch.setenv("HF_TOKEN", "env_wins")
    assert D.Credentials.load().hf_token == "env_wins"
    assert D.format_listings([]) == "No datasets found."
    out = D.format_listings([D.DatasetListing("a/b", "d" * 100, 7, [])])
    assert "1. a/b" in out and "Downloads: 7" in out and ("d" * 80 + "...") in out
    # remote loaders are served from the cache directory; nothing cached and no network -> DataError
    cache = D.make_classification(5, 2, 2, seed=0)
    os.makedirs(D.cache_dir(), exist_ok=True)
    with open(os.path.join(D.cache_dir(), "org_name_train.json"), "w") as f:
        f.write(D.dataset_to_cache_json(cache))
    got = D.load_huggingface("org/name", "train", 5)
    assert got.num_rows == 5 and got.get_float("f0").tolist() == cache.get_float("f0").tolist()
    rows = D.extract_rows_from_hf_json('{"rows":[{"row_idx":0,"row":{"text":"a","label":1}},{"row_idx":1,"row":{"text":"b","label":0}}]}')
    assert rows == [{"text": "a", "label": "1"}, {"text": "b", "label": "0"}]
    with pytest.raises(D.DataError):
        D.load_kaggle("x/y", "f.csv", D.Credentials())


# ------------------------------------------------------------------ offload
def test_ssd_tensor_format_and_store(tmp_path):
    t = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    s = offload.SsdTensor.write(t, str(tmp_path))
    raw = open(s.path(), "rb").read()
    assert raw[:4] == struct.pack("<I", 2) and raw[4:20] == struct.pack("<QQ", 2, 3) and raw[20:] == t.numpy().tobytes()
    assert s.size_bytes() == 4 + 16 + 24 and s.shape() == [2, 3] and torch.equal(s.load(), t)
    path = s.path()
    del s
    assert not os.path.exists(path)                      # the spill file dies with its handle
    cfg = offload.OffloadConfig().with_ssd_dir(str(tmp_path / "ssd")).with_hot_cache(4)
    cfg.ram_budget_bytes = 4 * 100 * 2 + 10              # room for two 100-float tensors
    store = offload.TieredStore.new(cfg)
    for i in range(4):
        store.insert(f"t{i}", torch.full((100,), float(i)))
    ram, ssd = store.tier_counts()
    assert ram == 2 and ssd == 2 and store.ram_usage() == 800 and store.ssd_usage() > 800
    assert store.tensors["t0"].tier() == offload.MemoryTier.Ssd           # the oldest went first
    assert float(store.get("t0").sum()) == 0.0 and float(store.get("t1")[0]) == 1.0
    assert store.ram_usage() <= cfg.ram_budget_bytes and store.get("nope") is None
    store.offload_all()
    assert store.tier_counts() == (0, 4) and store.ram_usage() == 0
    store.load_all()
    assert store.tier_counts() == (4, 0) and store.ram_usage() == 1600
    assert str(offload.MemoryTier.Ssd) == "SSD" and offload.OffloadConfig().with_ram_budget_gb(0.5).ram_budget_bytes == 512 * 1024 * 1024


def test_offload_model_round_trip(tmp_path):
    torch.manual_seed(0)
    model = nn.Sequential().add(nn.Linear(8, 16)).add(nn.ReLU()).add(nn.Linear(16, 4))
    x = torch.randn(3, 8)
    want = model(x).detach().clone()
    om = offload.OffloadModel(model, offload.OffloadConfig().with_ssd_dir(str(tmp_path)))
    assert om.ssd_usage() == 0 and om.ram_usage() == (8 * 16 + 16 + 16 * 4 + 4) * 4
    om.offload()
    assert om.ram_usage() == 0 and om.ssd_usage() > 0 and all(p.numel() == 0 for p in model.parameters())
    assert "SSD: 4" in om.memory_report()
    got = om.forward(x)
    assert torch.allclose(got, want, atol=1e-6) and not om.offloaded and "RAM: 4" in om.memory_report()


# ------------------------------------------------------------------ interactive / gui
def test_sparkline_and_commands():
    s = interactive.sparkline([10.0, 8.0, 5.0, 3.0, 1.0])
    assert len(s) == 5 and s[0] == "█" and s[-1] == "▁"
    assert set(interactive.sparkline([5.0, 5.0, 5.0])) == {"█"} and interactive.sparkline([]) == ""
    ses = interactive.Session.new()
    assert "New model" in interactive.process_command(ses, "model new")
    assert "Linear(4 -> 2)" in interactive.process_command(ses, "model add linear 4 2")
    assert ses.model is not None and ses.model_input_dim == 4 and ses.model_output_dim == 2
    ses2 = interactive.Session()
    out = interactive.process_command(ses2, "data synthetic 50 3 2")
    assert "synthetic" in out and ses2.dataset is not None and len(ses2.feature_columns) == 3 and ses2.target_column == "label"
    assert interactive.process_command(ses2, "info") == "model: false, dataset: true"
    assert interactive.process_command(ses2, "") == "" and interactive.process_command(ses2, "bogus") == ""


def test_repl_trains_a_model():
    script = "\n".join(["help", "model new", "model add linear 3 8", "model add relu", "model add linear 8 1", "model summary",
                        "data regression 64 3", "data columns", "data head 2", "train 30 0.05", "predict 1", "info", "nonsense", "tensor zeros 2 2",
                        "exit"]) + "\n"
    out = io.StringIO()
    interactive.run_repl(io.StringIO(script), out)
    text = out.getvalue()
    assert "Added Linear(3 -> 8)" in text and "Parameters: 4 tensors, 41 total elements" in text and "[target]" in text
    assert "Epoch  30" in text and "Training complete" in text and "Prediction for row 1" in text and "Unknown command: 'nonsense'" in text
    assert "Goodbye!" in text
    first = float(text.split("Epoch   1: loss =")[1].split()[0])
    last = float(text.split("Epoch  30: loss =")[1].split()[0])
    assert last < first


def test_dashboards(tmp_path):
    d = gui.ModelDashboard.new("MLP").layer("Linear", 10, 20, "he").layer("ReLU", 20, 20, "").layer("Linear", 20, 5, "he")
    h = d.render()
    assert "<html" in h and "Linear" in h and "Parameters" in h and d.param_count() == 10 * 20 + 20 + 20 * 5 + 5 and "#D94A4A" in h
    t = gui.TrainingDashboard.new("Run")
    assert "No data" in t.render()
    t.add_point(1, 3.0); t.add_point(2, 1.0)
    r = t.render()
    assert "<svg" in r and "polyline" in r and "66.7%" in r
    hm = gui.tensor_heatmap_html(torch.tensor([[1.0, 2.0], [3.0, 4.0]]), 100)
    assert hm.count("<td") == 4 and "hsl(240" in hm and "hsl(0" in hm and hm.count("</tr><tr>") == 1
    full = gui.full_dashboard("Full", gui.ModelDashboard("M").layer("Linear", 4, 8, "he"), t)
    assert "Architecture" in full and "Metrics" in full and full.count("<html") == 1
    m = nn.Sequential().add(nn.Linear(4, 8)).add(nn.ReLU()).add(nn.Linear(8, 2))
    assert gui.ModelDashboard.from_model("auto", m).param_count() == 4 * 8 + 8 + 8 * 2 + 2
    p = tmp_path / "dash.html"
    gui.launch(full, str(p))
    assert p.read_text() == full
    assert "polyline" in gui.TrainingDashboard.from_history("h", [3.0, 2.0, 1.0]).render()


# ------------------------------------------------------------------ BLAS / SIMD / fused / compiled / gpu surface (CPU path)
def test_blas_surface_cpu():
    torch.manual_seed(0)
    a, b = torch.randn(5, 7), torch.randn(7, 3)
    c = torch.zeros(15)
    blas.matmul(a.reshape(-1), b.reshape(-1), c, 5, 7, 3)
    assert torch.allclose(c.view(5, 3), a @ b, atol=1e-5)
    c2 = torch.ones(5, 3)
    blas.sgemm(blas.Transpose.Trans, blas.Transpose.Trans, 5, 3, 7, 2.0, a.t().contiguous(), 5, b.t().contiguous(), 7, 0.5, c2, 3)
    assert torch.allclose(c2, 2.0 * a @ b + 0.5, atol=1e-5)
    big = torch.zeros(5, 6)                                  # ldc > n: only the first 3 columns are written
    blas.sgemm(blas.Transpose.NoTrans, blas.Transpose.NoTrans, 5, 3, 7, 1.0, a, 7, b, 3, 0.0, big, 6)
    assert torch.allclose(big[:, :3], a @ b, atol=1e-5) and float(big[:, 3:].abs().sum()) == 0.0
    x, y = torch.randn(7), torch.ones(5)
    blas.sgemv(blas.Transpose.NoTrans, 5, 7, 2.0, a, 7, x, 1, 3.0, y, 1)
    assert torch.allclose(y, 2 * a @ x + 3, atol=1e-5)
    yt = torch.zeros(7)
    blas.sgemv(blas.Transpose.Trans, 5, 7, 1.0, a, 7, torch.ones(5), 1, 0.0, yt, 1)
    assert torch.allclose(yt, a.sum(0), atol=1e-5)
    assert float(blas.sdot(3, torch.tensor([1.0, 9, 2, 9, 3]), 2, torch.tensor([1.0, 1, 1]), 1)) == 6.0
    assert float(blas.snrm2(2, torch.tensor([3.0, 4.0]))) == 5.0
    v = torch.ones(4)
    blas.saxpy(4, 2.0, torch.arange(4.0), v); blas.sscal(4, 0.5, v)
    assert v.tolist() == [0.5, 1.5, 2.5, 3.5]
    w = torch.zeros(4); blas.scopy(4, v, w)
    assert torch.equal(w, v)
    cs = torch.zeros(5, 3); blas.gemm_strassen(a, b, cs, 5, 7, 3)
    assert torch.allclose(cs, a @ b, atol=1e-5)


def test_simd_fused_surface_cpu():
    a, b = torch.tensor([1.0, -2.0, 3.0]), torch.tensor([4.0, 5.0, -6.0])
    out = torch.zeros(3)
    assert simd.simd_add(a, b, out) is out and out.tolist() == [5.0, 3.0, -3.0]
    assert simd.simd_mul(a, b).tolist() == [4.0, -10.0, -18.0] and simd.simd_relu(a).tolist() == [1.0, 0.0, 3.0]
    assert simd.simd_scale(a, 2.0).tolist() == [2.0, -4.0, 6.0] and float(simd.simd_sum(a)) == 2.0
    c = torch.zeros(4)
    simd.simd_matmul(torch.tensor([1.0, 2, 3, 4]), torch.tensor([1.0, 0, 0, 1]), c, 2, 2, 2)
    assert c.tolist() == [1.0, 2.0, 3.0, 4.0] and isinstance(simd.simd_features(), str)
    x = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    w = torch.tensor([[1.0, 0.0, 0.0], [0.0, -1.0, 0.0]])
    bias = torch.tensor([0.1, 0.2])
    assert torch.allclose(fused.fused_linear(x, w, bias, fused.FusedActivation.ReLU), torch.tensor([[1.1, 0.0], [4.1, 0.0]]))
    assert torch.allclose(fused.fused_linear(x, w, None, fused.FusedActivation.None_), x @ w.t())
    g = fused.fused_linear(x, w, bias, fused.FusedActivation.GELU)
    assert torch.allclose(g, torch.nn.functional.gelu(x @ w.t() + bias, approximate="tanh"), atol=1e-6)
    s = fused.fused_linear(x, w, bias, fused.FusedActivation.Sigmoid)
    assert torch.allclose(s, torch.sigmoid(x @ w.t() + bias), atol=1e-6) and not s.requires_grad
    idx, wts = fused.sparse_topk_route(torch.tensor([0.1, 2.0, 1.0, -1.0, 3.0, 0.0, 0.5, 0.2]), 2, 4, 2)
    assert idx.tolist() == [1, 2, 0, 2] and torch.allclose(wts.view(2, 2).sum(-1), torch.ones(2))
    assert float(wts[0]) == pytest.approx(math.exp(2) / (math.exp(2) + math.exp(1)))


def test_compiled_mlp_cpu():
    m = compiled.CompiledMLP([(4, 8), (8, 2)], 16, 0.01, device="cpu")
    # the reference's LCG initialisation: first weight of a (4 -> 8) layer
    seed = (4 * 31 + 8) & 0xFFFFFFFF
    x1 = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
    want = ((x1 >> 8) / 16777216.0 - 0.5) * 2.0 * math.sqrt(2.0 / 4)
    assert float(m.weights()[0].reshape(-1)[0]) == pytest.approx(want, rel=1e-6) and float(m.biases()[0].abs().sum()) == 0.0
    g = torch.Generator().manual_seed(0)
    x = torch.randn(16, 4, generator=g)
    y = x[:, :2] * 0.5
    l0 = m.step(x.reshape(-1).tolist(), y.reshape(-1).tolist())
    for _ in range(200):
        l1 = m.step(x, y)
    assert l1 < 0.2 * l0 and m.t == 201 and tuple(m.forward(x).shape) == (16, 2)
    # the loss is the mean of squared errors
    m2 = compiled.CompiledMLP.new([(4, 2)], 16, 0.0)
    assert m2.step(x, y) == pytest.approx(float(((m2.forward(x) - y) ** 2).mean()), rel=1e-5)


def test_gpu_surface_cpu(tmp_path):
    nv = gpu.TileConfig.nvidia()
    assert (nv.bm, nv.bn, nv.bk, nv.warp_size) == (128, 256, 64, 32) and nv.shared_mem_bytes() == (128 * 64 + 64 * 256) * 2
    assert gpu.TileConfig.amd().warp_size == 64 and gpu.TileConfig.cpu().arithmetic_intensity() > 0
    assert gpu.TileConfig.for_backend(gpu.GpuBackendKind.WebGpu) == gpu.TileConfig.cpu()
    assert gpu.detect_backend() in (gpu.GpuBackendKind.Nvidia, gpu.GpuBackendKind.Cpu) and gpu_kernels.active_backend() is gpu.active_backend()
    rep = gpu.backend_report()
    assert "[ACTIVE]" in rep and "BM=128" in rep and "Arith intensity" in rep
    src = gpu.kernel_source(gpu.GpuBackendKind.Nvidia)
    assert "tcgen05" in src and "__global__" in src and "No kernel" in gpu.kernel_source(gpu.GpuBackendKind.Apple)
    files = gpu.extract_kernels(str(tmp_path / "k"))
    assert any(f.endswith("gemm_sm100.cu") for f in files) and all(os.path.exists(f) for f in files)
    with pytest.raises(ValueError):
        gpu.set_backend(gpu.GpuBackendKind.Amd)
    a, b = torch.randn(4, 5), torch.randn(5, 3)
    c, used = gpu.kernel_matmul_with_backend(a, b, gpu.GpuBackendKind.Cpu)
    assert used is gpu.GpuBackendKind.Cpu and torch.allclose(c, a @ b, atol=1e-5)
    if not torch.cuda.is_available():
        assert not gpu.has_gpu() and gpu.gpu() is None and gpu.GpuBackend.new() is None
        assert torch.allclose(gpu.gpu_matmul(a, b), a @ b, atol=1e-5)
        w, bias = torch.randn(3, 5), torch.randn(3)
        assert torch.allclose(gpu.gpu_linear(a, w, bias, True), torch.relu(a @ w.t() + bias), atol=1e-5)
        q = torch.randn(6, 8)
        assert torch.allclose(gpu.gpu_attention(q, q, q, 0.3), torch.softmax(q @ q.t() * 0.3, -1) @ q, atol=1e-5)
        assert torch.equal(gpu.gpu_relu(torch.tensor([-1.0, 2.0])), torch.tensor([0.0, 2.0]))
        assert torch.equal(gpu.gpu_add(a, a), a + a) and torch.equal(gpu.gpu_mul(a, a), a * a)


def test_core_ops_bench_runs_every_group_on_cpu():
    """benches/core_ops.py (the counterpart of the reference's criterion groups) runs end to end on the CPU path."""
    import importlib.util
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benches", "core_ops.py")
    spec = importlib.util.spec_from_file_location("core_ops_bench", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert set(mod.GROUPS) == {"matmul", "simd_matmul", "attention", "gemm_train", "int8_vs_fp32", "blas_sgemm", "dropout",
                               "fused_linear", "elementwise", "backward"}
    b = mod.Bench("cpu", 1, 1)
    for fn in mod.GROUPS.values():
        fn(b, True)
    assert len(b.rows) >= 20 and all(t > 0 for _, _, t in b.rows)


@pytest.mark.parametrize("script,args", [("basic.py", []), ("xor.py", []), ("bench_train.py", ["--scale", "0.01"]), ("bench_compiled.py", ["--iters", "2"])])
def test_examples_run_on_cpu(script, args):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, os.path.join(root, "examples", script), *args], capture_output=True, text=True, timeout=600,
                       cwd=os.path.join(root, "examples"), env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip()
