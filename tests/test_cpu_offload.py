"""offload.py, one test per behaviour of rust-nn src/offload.rs:560-700: tensors spilled to files and read back,
the RAM budget's eviction of the coldest tensor, a model whose weights come back from disk for its forward."""
import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200.offload import MemoryTier, OffloadConfig, OffloadModel, SsdTensor, TieredStore, TieredTensor


def test_ssd_tensor_round_trip(tmp_path):
    t = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    s = SsdTensor.write(t, str(tmp_path))
    assert tuple(s.shape()) == (2, 3)
    assert torch.equal(s.load(), t)


def test_ssd_tensor_large(tmp_path):
    t = torch.randn(128, 256)
    back = SsdTensor.write(t, str(tmp_path)).load()
    assert tuple(back.shape) == (128, 256) and torch.equal(back, t)


def test_tiered_tensor_offload_and_load(tmp_path):
    tt = TieredTensor.from_tensor(torch.tensor([10.0, 20.0, 30.0]))
    assert tt.tier() == MemoryTier.Ram
    tt.offload_to_ssd(str(tmp_path))
    assert tt.tier() == MemoryTier.Ssd
    tt.load_to_ram()
    assert tt.tier() == MemoryTier.Ram
    assert tt.get().tolist() == [10.0, 20.0, 30.0]


def test_store_evicts_to_stay_under_the_ram_budget(tmp_path):
    store = TieredStore.new(OffloadConfig(ram_budget_bytes=120, ssd_dir=str(tmp_path), hot_cache_size=1))
    store.insert("a", torch.full((20,), 1.0))                     # 80 bytes
    store.insert("b", torch.full((20,), 2.0))                     # 80 more: "a" has to go
    ram, ssd = store.tier_counts()
    assert ssd >= 1 and ram + ssd == 2
    assert store.ram_usage() <= 120


def test_store_get_loads_from_ssd(tmp_path):
    store = TieredStore.new(OffloadConfig(ram_budget_bytes=0, ssd_dir=str(tmp_path), hot_cache_size=10))
    store.insert("x", torch.tensor([42.0, 43.0]))
    store.offload("x")
    assert store.tier_counts() == (0, 1)
    assert store.get("x").tolist() == [42.0, 43.0]
    assert store.get("missing") is None


def test_offload_model_round_trip(tmp_path):
    torch.manual_seed(0)
    model = nn.Sequential().add(nn.Linear(8, 16)).add(nn.ReLU()).add(nn.Linear(16, 4))
    x = torch.randn(2, 8)
    want = model(x).detach().clone()
    om = OffloadModel(model, OffloadConfig(ram_budget_bytes=0, ssd_dir=str(tmp_path), hot_cache_size=10))
    om.offload()
    assert om.ssd_usage() > 0
    y = om.forward(x)                                             # the weights come back from their files first
    assert tuple(y.shape) == (2, 4) and torch.allclose(y.detach(), want, atol=1e-6)


def test_memory_report_names_tiers_and_tensors(tmp_path):
    om = OffloadModel(nn.Sequential().add(nn.Linear(4, 8)), OffloadConfig().with_ssd_dir(str(tmp_path)))
    report = om.memory_report()
    assert "RAM" in report and "tensors" in report


def test_config_builder():
    c = OffloadConfig().with_ram_budget_gb(8.0).with_hot_cache(64)
    assert c.ram_budget_bytes == 8 * 1024 ** 3 and c.hot_cache_size == 64
