"""Sectioned visualisation configuration: validation rules, builder, loaders, effect on the visualizer."""
import json

import pytest
import torch

from ml_framework_b200.obs import vis_config as VC
from ml_framework_b200.obs.events import MemoryStorageBackend


def test_validator_errors_and_warnings():
    v = VC.ConfigurationValidator()
    assert v.validate(VC.FullVisualizationConfiguration()).is_valid and not v.validate(None).is_valid
    c = VC.FullVisualizationConfiguration()
    c.storage.log_directory = " "; c.storage.write_buffer_size = 0; c.storage.flush_interval_s = 0; c.storage.backend_type = "sql"
    c.logging.histogram_bin_count = 0; c.logging.default_smoothing_window = -1
    c.profiling.max_stored_operations = 0
    c.memory_profiling.max_stack_trace_depth = 0; c.memory_profiling.snapshot_interval_ms = 0
    c.gpu_tracking.sampling_interval_ms = 0
    c.event_collection.buffer_capacity = 10; c.event_collection.batch_size = 20; c.event_collection.max_queue_length = 0
    r = v.validate(c)
    assert len(r.errors) == 12 and "12 error(s)" in r.summary() and any("batch_size cannot be larger than buffer_capacity" in e for e in r.errors)
    w = VC.FullVisualizationConfiguration()
    w.storage.write_buffer_size = 200000; w.storage.flush_interval_s = 600
    w.logging.histogram_bin_count = 5000; w.logging.default_smoothing_window = 5000
    w.profiling.max_stored_operations = 10 ** 6; w.profiling.profile_cpu = w.profiling.profile_gpu = False
    w.memory_profiling.max_stack_trace_depth = 80; w.memory_profiling.snapshot_interval_ms = 10; w.memory_profiling.capture_stack_traces = True
    w.gpu_tracking.enable_gpu_tracking = True; w.gpu_tracking.sampling_interval_ms = 10
    w.gpu_tracking.track_power = w.gpu_tracking.track_temperature = False
    w.event_collection.buffer_capacity = 200000
    r = v.validate(w)
    assert r.is_valid and len(r.warnings) == 12
    c.storage = None
    assert v.validate(c).errors == ["storage configuration cannot be None"]
    with pytest.raises(ValueError, match="invalid"):
        v.validate_or_raise(c)


def test_builder_and_loaders(tmp_path):
    b = (VC.VisualizationConfigurationBuilder().with_storage_directory(str(tmp_path / "runs")).with_storage_backend("memory")
         .with_log_prefix("train/").with_histogram_bin_count(12).enable_gpu_profiling(False).with_max_stored_operations(50)
         .enable_memory_profiling().with_memory_snapshot_interval_ms(500).enable_gpu_tracking().with_gpu_sampling_interval_ms(250)
         .enable_async_event_collection(False).with_event_buffer_capacity(64).with_event_batch_size(8).with_verbose_logging())
    c = b.build()
    assert c.logging.scalar_log_prefix == "train/" and c.event_collection.batch_size == 8 and c.verbose_logging and not c.profiling.profile_gpu
    flat = c.to_flat()
    assert flat.storage == "memory" and flat.histogram_bins == 12 and flat.buffer_capacity == 64 and not flat.async_collection
    with pytest.raises(ValueError):
        VC.VisualizationConfigurationBuilder().with_event_batch_size(0).build()
    cfg, res = VC.VisualizationConfigurationBuilder().with_histogram_bin_count(-1).build_with_validation()
    assert not res.is_valid and VC.VisualizationConfigurationBuilder().with_histogram_bin_count(-1).build_without_validation().logging.histogram_bin_count == -1
    L = VC.SectionedConfigurationLoader
    p = tmp_path / "vis.json"
    L.save(c, str(p))
    again = L.from_file(str(p))
    assert again == c
    env = {"MLFRAMEWORK_VISUALIZATION_LOGGING__HISTOGRAM_BIN_COUNT": "20", "MLFRAMEWORK_VISUALIZATION_IS_ENABLED": "off",
           "MLFRAMEWORK_VISUALIZATION_STORAGE__FLUSH_INTERVAL_S": "2.5", "OTHER": "x"}
    over = L.load(str(p), env)
    assert over.logging.histogram_bin_count == 20 and over.is_enabled is False and over.storage.flush_interval_s == 2.5
    with pytest.raises(KeyError):
        L.from_environment(env={"MLFRAMEWORK_VISUALIZATION_LOGGING__NOPE": "1"})
    with pytest.raises(ValueError):
        L.from_environment(env={"MLFRAMEWORK_VISUALIZATION_VERBOSE_LOGGING": "maybe"})
    with pytest.raises(KeyError, match="unknown logging settings"):
        L.from_json(json.dumps({"logging": {"colour": 1}}))
    with pytest.raises(KeyError, match="unknown configuration section"):
        L.from_json(json.dumps({"plots": {}}))
    with pytest.raises(ValueError):
        L.load(env={"MLFRAMEWORK_VISUALIZATION_EVENT_COLLECTION__BATCH_SIZE": "0"})
    with pytest.raises(FileNotFoundError):
        L.from_file(str(tmp_path / "none.json"))


def test_make_visualizer_applies_logging_switches():
    c = (VC.VisualizationConfigurationBuilder().with_storage_backend("memory").with_log_prefix("run1/")
         .enable_async_event_collection(False).build())
    c.logging.log_histograms = False
    c.logging.log_hyperparameters = False
    c.profiling.enable_profiling = False
    backend = MemoryStorageBackend()
    v = VC.make_visualizer(c, backend)
    v.log_scalar("loss", 1.5, 3)
    v.log_histogram("w", torch.randn(10))
    v.log_hyperparameters({"lr": 1e-3})
    v.log_text("note", "hello")
    with v.start_profile("fwd"):
        pass
    v.flush()
    names = [e.name for e in backend.events]
    assert "run1/loss" in names and "note" in names and "w" not in names and "hparams" not in names
    assert "run1/loss" in v.scalars.series and not v.profiler.results() and v.full_config is c
    v.close()
    off = VC.VisualizationConfigurationBuilder().with_storage_backend("memory").with_scalar_logging(False).enable_async_event_collection(False).build()
    v2 = VC.make_visualizer(off)
    v2.log_scalar("loss", 1.0)
    assert not v2.scalars.series
    v2.close()
