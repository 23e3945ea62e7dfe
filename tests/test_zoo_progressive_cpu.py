"""Progressive loading: lazy layers on meta, strategies, unload policies, events, both file formats."""
import threading

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.modelzoo import progressive as PG
from ml_framework_b200.modelzoo.serialization import ModelSerializer


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.inp = nn.Linear(8, 16)
        self.blocks = nn.ModuleList([nn.Sequential(nn.Linear(16, 16), nn.BatchNorm1d(16)) for _ in range(3)])
        self.act = nn.ReLU()
        self.out = nn.Linear(16, 4)

    def forward(self, x):
        x = self.inp(x)
        for b in self.blocks:
            x = self.act(b(x))
        return self.out(x)


def _reference():
    torch.manual_seed(0)
    m = Net().eval()
    for b in m.blocks:
        b[1].running_mean.normal_(); b[1].running_var.uniform_(0.5, 2.0)
    return m


def test_load_order_dependencies_and_architecture_guess():
    o = PG.LayerLoadOrder.for_architecture("GPT-style transformer")
    assert o.architecture_type is PG.ModelArchitectureType.TRANSFORMER
    assert PG.LayerLoadOrder.for_architecture("ResNet50").architecture_type is PG.ModelArchitectureType.CNN
    assert PG.LayerLoadOrder.for_architecture("lstm-lm").architecture_type is PG.ModelArchitectureType.RNN
    for n in ("head", "b1", "b0", "embed"):
        o.add_layer(n)
    o.add_dependency("head", "b1"); o.add_dependency("b1", "b0"); o.add_dependency("b0", "embed"); o.add_dependency("b0", "embed")
    assert o.get_load_order() == ["embed", "b0", "b1", "head"]
    m = PG.LayerLoadOrder.from_model(Net())
    assert m.get_load_order() == ["inp", "blocks.0.0", "blocks.0.1", "blocks.1.0", "blocks.1.1", "blocks.2.0", "blocks.2.1", "out"]


def test_memory_manager_policies():
    now = [0.0]
    lru = PG.MemoryManager(PG.ProgressiveLoadOptions(unload_strategy=PG.UnloadStrategy.LRU, max_loaded_layers=2), lambda: now[0])
    for i, n in enumerate("abc"):
        now[0] = i
        lru.register_layer(n, 100)
    assert lru.has_memory_pressure() and lru.get_layers_to_unload() == ["a"]
    lru.record_access("a")
    assert lru.get_layers_to_unload() == ["b"] and lru.get_layers_to_unload(keep=("b",)) == ["c"]
    assert lru.unregister_layer("b") == 100 and not lru.has_memory_pressure() and lru.total_loaded_bytes == 200
    assert lru.get_memory_info()["a"].last_access_time == 2 and lru.unregister_layer("zz") == 0
    mp = PG.MemoryManager(PG.ProgressiveLoadOptions(unload_strategy=PG.UnloadStrategy.MEMORY_PRESSURE, memory_pressure_threshold=250))
    for n, sz in (("a", 100), ("b", 100), ("c", 100), ("d", 100)):
        mp.register_layer(n, sz)
    assert mp.has_memory_pressure() and mp.get_layers_to_unload() == ["a", "b"] and mp.get_layers_to_unload(count=1) == ["a"]
    never = PG.MemoryManager(PG.ProgressiveLoadOptions())
    never.register_layer("a", 10 ** 12)
    assert not never.has_memory_pressure() and never.get_layers_to_unload() == []
    mp.clear()
    assert mp.loaded_layer_count == 0 and mp.total_loaded_bytes == 0


@pytest.mark.parametrize("fmt", ["torch", "zoo"])
def test_on_demand_loading_from_meta_matches_the_full_model(tmp_path, fmt):
    ref = _reference()
    path = str(tmp_path / "w.bin")
    if fmt == "torch":
        torch.save(ref.state_dict(), path)
    else:
        ModelSerializer().serialize_to_file(ref.state_dict(), path)
    model, loader = PG.load_progressive(lambda: Net().eval(), path)
    assert all(p.is_meta for p in model.parameters()) and loader.get_loading_progress() == 0.0
    names, progress, full = [], [], []
    loader.on_layer_loaded.append(names.append)
    loader.on_progress_changed.append(progress.append)
    loader.on_fully_loaded.append(lambda: full.append(True))
    x = torch.randn(5, 8)
    torch.testing.assert_close(model(x), ref(x))
    assert names == loader.context.layer_load_order.get_load_order() and progress[-1] == 1.0 and full == [True]
    assert loader.is_fully_loaded() and loader.wait_for_fully_loaded(10) and not any(p.is_meta for p in model.parameters())
    assert loader.context.memory_manager.total_loaded_bytes == sum(l.size_in_bytes for l in loader.lazy_layers.values())
    torch.testing.assert_close(model(x), ref(x))                     # second pass loads nothing
    assert len(names) == 8 and full == [True]
    loader.close()
    assert isinstance(loader.source, PG.TorchFileSource if fmt == "torch" else PG.ZooFileSource)


def test_lru_unload_keeps_at_most_n_layers_and_reloads():
    ref = _reference()
    src = PG.DictSource(ref.state_dict())
    with torch.device("meta"):
        model = Net().eval()
    opts = PG.ProgressiveLoadOptions(unload_strategy=PG.UnloadStrategy.LRU, max_loaded_layers=2)
    loader = PG.ProgressiveModelLoader(model, src, opts)
    peak = [0]
    loader.on_layer_loaded.append(lambda n: peak.__setitem__(0, max(peak[0], loader.context.memory_manager.loaded_layer_count)))
    x = torch.randn(3, 8)
    torch.testing.assert_close(model(x), ref(x))
    mm = loader.context.memory_manager
    assert mm.loaded_layer_count == 2 and peak[0] <= 3 and sorted(loader.context.loaded_layers) == ["blocks.2.1", "out"]
    assert model.inp.weight.is_meta and not model.out.weight.is_meta and loader.is_fully_loaded()
    n_reads = len(src.reads)
    torch.testing.assert_close(model(x), ref(x))                     # evicted layers come back
    assert len(src.reads) > n_reads and mm.loaded_layer_count == 2
    assert model.blocks[0][1].running_mean.is_meta                    # buffers leave too
    loader.close()


def test_memory_pressure_unload_by_bytes():
    ref = _reference()
    with torch.device("meta"):
        model = Net().eval()
    one_block = (16 * 16 + 16) * 4
    opts = PG.ProgressiveLoadOptions(unload_strategy=PG.UnloadStrategy.MEMORY_PRESSURE, memory_pressure_threshold=3 * one_block)
    loader = PG.ProgressiveModelLoader(model, PG.DictSource(ref.state_dict()), opts)
    x = torch.randn(3, 8)
    torch.testing.assert_close(model(x), ref(x))
    assert loader.context.memory_manager.total_loaded_bytes <= 3 * one_block + loader.get_layer("out").size_in_bytes
    loader.close()


@pytest.mark.parametrize("strategy", [PG.LayerLoadingStrategy.SEQUENTIAL, PG.LayerLoadingStrategy.PARALLEL])
def test_background_strategies_finish_without_a_forward_pass(strategy):
    ref = _reference()
    with torch.device("meta"):
        model = Net().eval()
    loader = PG.ProgressiveModelLoader(model, PG.DictSource(ref.state_dict()), PG.ProgressiveLoadOptions(strategy=strategy, max_concurrent_loads=3))
    assert loader.wait_for_fully_loaded(20000) and not any(p.is_meta for p in model.parameters())
    x = torch.randn(2, 8)
    torch.testing.assert_close(model(x), ref(x))
    assert loader.context.get_next_layers_to_load() == []
    loader.close()


def test_prefetch_strategy_loads_ahead_and_next_layer_queries():
    ref = _reference()
    gate = threading.Event()

    class Slow(PG.DictSource):
        def read(self, names):
            if any(n.startswith("blocks.0.0") for n in names):
                gate.set()
            return super().read(names)

    with torch.device("meta"):
        model = Net().eval()
    opts = PG.ProgressiveLoadOptions(strategy=PG.LayerLoadingStrategy.PREFETCH, prefetch_count=2)
    loader = PG.ProgressiveModelLoader(model, Slow(ref.state_dict()), opts)
    assert loader.context.get_next_layers_to_load() == ["inp", "blocks.0.0"]
    assert loader.context.get_next_layers_to_load("blocks.2.0") == ["blocks.2.1", "out"]
    model.inp(torch.randn(1, 8))                                    # touching the first layer starts the next two
    assert gate.wait(10)
    for f in loader.prefetch_next_layers("inp"):
        f.result(10)
    assert loader.context.is_layer_loaded("blocks.0.0") and loader.context.is_layer_loaded("blocks.0.1")
    x = torch.randn(2, 8)
    torch.testing.assert_close(model(x), ref(x))
    with pytest.raises(KeyError):
        loader.prefetch_layer("nope")
    loader.close()
    par = PG.ProgressiveLoadContext(None, "cpu", PG.ProgressiveLoadOptions(strategy=PG.LayerLoadingStrategy.PARALLEL, max_concurrent_loads=3),
                                    loader.context.layer_load_order)
    par.mark_layer_loaded("inp", 1)
    assert par.get_next_layers_to_load() == ["blocks.0.0", "blocks.0.1", "blocks.1.0"]


def test_strict_missing_keys_shape_mismatch_and_dtype_cast():
    ref = _reference()
    sd = dict(ref.state_dict())
    part = {k: v for k, v in sd.items() if not k.startswith("out.")}
    with torch.device("meta"):
        m1 = Net()
    with pytest.raises(KeyError):
        PG.ProgressiveModelLoader(m1, PG.DictSource(part))
    with torch.device("meta"):
        m2 = Net()
    loose = PG.ProgressiveModelLoader(m2, PG.DictSource(part), strict=False)
    assert sorted(loose.missing_keys) == ["out.bias", "out.weight"]
    loose.close()
    bad = dict(sd); bad["inp.weight"] = torch.zeros(3, 3)
    with torch.device("meta"):
        m3 = Net()
    l3 = PG.ProgressiveModelLoader(m3, PG.DictSource(bad))
    with pytest.raises(ValueError, match="shape"):
        l3.get_layer("inp").ensure_loaded()
    l3.close()
    with torch.device("meta"):
        m4 = Net().eval()
    l4 = PG.ProgressiveModelLoader(m4, PG.DictSource(sd), dtype=torch.bfloat16)
    l4.load_all()
    assert m4.inp.weight.dtype == torch.bfloat16 and m4.blocks[0][1].num_batches_tracked.dtype == torch.int64
    assert l4.get_layer("inp").size_in_bytes == (8 * 16 + 16) * 2 and l4.get_layer("inp").unload() and not l4.get_layer("inp").unload()
    l4.close()


def test_zoo_load_progressive_gives_the_same_logits(tmp_path):
    from ml_framework_b200.modelzoo import zoo as Z
    z = Z.ModelZoo(str(tmp_path / "cache"))
    torch.manual_seed(0)
    m = z.load("llama-tiny", pretrained=False).eval()
    z.save(m, Z.ModelInfo("mine", "llama", z.registry.get("llama-tiny").config, version="2.0.0"), str(tmp_path / "w.pt"))
    lazy, loader = z.load_progressive("mine", options=PG.ProgressiveLoadOptions(unload_strategy=PG.UnloadStrategy.LRU, max_loaded_layers=3))
    lazy.eval()
    assert loader.context.layer_load_order.architecture_type is PG.ModelArchitectureType.TRANSFORMER
    ids = torch.randint(0, 100, (2, 16))
    with torch.no_grad():
        torch.testing.assert_close(lazy(ids), m(ids))
    assert loader.context.memory_manager.loaded_layer_count <= 3 and loader.is_fully_loaded()
    # the output projection is a parameter of the model itself: it lives in the pinned root layer
    assert PG.ROOT_LAYER in loader.context.loaded_layers and not lazy.lm_head.is_meta and lazy.embed.weight.is_meta
    loader.close()
    with pytest.raises(ValueError):
        z.load_progressive("llama-tiny")
