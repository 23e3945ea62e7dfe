"""Model-zoo bookkeeping types, card validation and the registry builder."""
import json

import pytest
import torch

from ml_framework_b200.modelzoo import config as C
from ml_framework_b200.modelzoo import zoo as Z


def _card(**kw):
    base = dict(name="m", architecture="mlp", config={}, version="1.0.0")
    base.update(kw)
    return Z.ModelInfo(**base)


def test_format_bytes_progress_and_cache_records():
    assert C.format_bytes(0) == "0 B" and C.format_bytes(1536) == "1.5 KB" and C.format_bytes(5 << 30) == "5 GB"
    p = C.DownloadProgress(512, 2048, "http://x", 256.0)
    assert p.progress_percentage == 0.25 and p.progress_percentage_text == "25.0%" and p.estimated_time_remaining_s == 6.0
    assert p.bytes_downloaded_text == "512 B" and p.total_bytes_text == "2 KB" and p.download_speed_text == "256 B/s"
    assert C.DownloadProgress().progress_percentage == 0.0 and C.DownloadProgress().estimated_time_remaining_s is None
    now, seen = [0.0], []
    track = C.DownloadProgress.tracker("u", seen.append, clock=lambda: now[0])
    track(0, 1000)
    now[0] = 2.0
    track(500, 1000)
    assert seen[-1].download_speed == 250.0 and seen[-1].current_url == "u"
    m = C.CacheMetadata("a", "1.0.0", 10, checksum="ab")
    m.record_access(now=5.0)
    back = C.CacheMetadata.from_json(m.to_json())
    assert back == m and back.access_count == 1 and back.last_accessed == 5.0
    st = C.CacheStatistics()
    st.record_hit(); st.record_miss(); st.record_hit()
    assert st.cache_hit_rate == pytest.approx(2 / 3) and "2 hits of 3 loads" in st.summary()
    assert C.TaskType.TEXT_GENERATION.value == "causal-lm" and C.ModelZooConfiguration().cache_enabled
    assert C.CacheConfiguration().lock_timeout_ms == 30_000


def test_cache_statistics_from_real_fetches(tmp_path):
    z = Z.ModelZoo(str(tmp_path / "cache"))
    torch.manual_seed(0)
    m = z.load("llama-tiny", pretrained=False)
    z.save(m, Z.ModelInfo("a", "llama", z.registry.get("llama-tiny").config, version="1.0.0"), str(tmp_path / "a.pt"))
    z.save(m, Z.ModelInfo("b", "llama", z.registry.get("llama-tiny").config, version="1.0.0"), str(tmp_path / "b.pt"))
    for name in ("a", "b", "a", "a"):
        z.downloads.fetch(z.registry.get(name))
    st = C.cache_statistics(z.cache, top=1)
    assert st.total_models == 2 and st.total_loads == 4 and st.cache_hits == 2 and st.cache_hit_rate == 0.5
    assert st.most_recently_used[0].model_name == "a" and st.most_recently_used[0].access_count == 3
    assert st.least_recently_used[0].model_name == "b" and st.total_cache_size == 2 * st.most_recently_used[0].file_size


def test_metadata_validator_rules():
    V = C.ModelMetadataValidator
    assert V.is_valid(_card()) and V.validate(None) == ["metadata cannot be None"]
    bad = _card(name=" ", version="1.0", source="ht!tp://x y", sha256="abc", file_size=-1,
                metrics={"accuracy": 1.2, "top5": -0.1, "perplexity": -3.0, "loss": float("nan"), "latency_ms": 3.0})
    errs = V.validate(bad)
    for piece in ("name is required", "semantic versioning", "not a valid URL", "64-character", "file size",
                  "'accuracy' has value 1.2", "'top5'", "'perplexity' has negative", "'loss' is not a number"):
        assert any(piece in e for e in errs), piece
    assert not any("latency_ms" in e for e in errs)
    assert V.is_valid(_card(version="2.1.0-rc.1+build5", source="/plain/path.pt", sha256="a" * 64))
    assert any("needs a config" in e for e in V.validate(_card(architecture="gpt")))
    assert any("cannot be negative" in e for e in V.validate(_card(architecture="gpt", config={"n_layers": -1})))
    with pytest.raises(ValueError, match="semantic"):
        V.validate_or_raise(_card(version="x"))


def test_registry_builder_sources_validation_and_duplicates(tmp_path):
    d = tmp_path / "cards"
    d.mkdir()
    (d / "one.json").write_text(json.dumps({"name": "one", "architecture": "mlp", "config": {}, "version": "1.0.0", "tags": ["t"]}))
    (d / "many.json").write_text(json.dumps([{"name": "two", "architecture": "mlp", "config": {}, "version": "1.0.0"},
                                             {"name": "two", "architecture": "mlp", "config": {}, "version": "1.1.0"}]))
    b = C.RegistryBuilder().add_from_directory(str(d)).add(_card(name="three"))
    assert b.count == 4
    reg = b.build()
    assert reg.get("two").version == "1.1.0" and reg.get("one").tags == ("t",) and len(reg.list()) == 4
    with pytest.raises(ValueError, match="appears twice"):
        C.RegistryBuilder().add_range([_card(), _card()]).build()
    with pytest.raises(ValueError, match="semantic"):
        C.RegistryBuilder().add(_card(version="v1")).build()
    assert C.RegistryBuilder().add(_card(version="v1")).build(validate=False).get("m").version == "v1"
    (d / "broken.json").write_text(json.dumps({"name": "x", "architecture": "mlp", "config": {}, "colour": "red"}))
    with pytest.raises(ValueError, match="colour"):
        C.RegistryBuilder().add_from_json_file(str(d / "broken.json"))
    with pytest.raises(FileNotFoundError):
        C.RegistryBuilder().add_from_directory(str(tmp_path / "none"))
    b.clear()
    assert b.count == 0


def test_latest_version_ordering_handles_prereleases_and_odd_strings():
    reg = Z.ZooRegistry()
    for v in ("1.9.0", "1.10.0-rc.1", "1.10.0", "nightly", "1.2"):
        reg.register(_card(version=v))
    assert reg.get("m").version == "1.10.0"
    only = Z.ZooRegistry()
    only.register(_card(version="nightly"))
    assert only.get("m").version == "nightly"
