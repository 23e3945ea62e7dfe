"""Registry plug-ins, authentication, configuration from the environment, extensions, discovery with reload."""
import json
import os

import pytest

from ml_framework_b200.modelzoo import errors as E
from ml_framework_b200.modelzoo import plugins as P
from ml_framework_b200.modelzoo.zoo import ModelInfo, ZooRegistry


def _info(name="m", version="1.0.0", **kw):
    return ModelInfo(name=name, architecture="mlp", config={}, version=version, **kw)


def test_authentication_headers_and_configuration_loader():
    h = {}
    P.ApiKeyAuthentication("k1", "X-Key").authenticate(h)
    P.TokenAuthentication("t1").authenticate(h)
    assert h == {"X-Key": "k1", "Authorization": "Bearer t1"}
    P.BasicAuthentication("u", "p").authenticate(h)
    assert h["Authorization"] == "Basic dTpw"
    P.CustomAuthentication(lambda hd: hd.update({"X-Sig": "s"}), "Sig").authenticate(h)
    assert h["X-Sig"] == "s"
    with pytest.raises(ValueError):
        P.ApiKeyAuthentication("")
    env = {"REG_REGISTRY_URL": "http://r", "REG_MAX_RETRIES": "7", "REG_ENABLE_CACHING": "false", "REG_HTTP_TIMEOUT_SECONDS": "x",
           "REG_AUTHENTICATION_TYPE": "basic", "REG_USERNAME": "u", "REG_PASSWORD": "p"}
    cfg = P.PluginConfigurationLoader.load_from_environment(P.AuthenticatedPluginConfiguration, "REG", env)
    assert cfg.registry_url == "http://r" and cfg.max_retries == 7 and cfg.enable_caching is False and cfg.http_timeout_seconds == 300
    assert isinstance(P.authentication_from(cfg), P.BasicAuthentication) and P.authentication_from(P.PluginConfigurationBase()) is None
    cfg.set_custom_property("region", "eu")
    assert cfg.get_custom_property("region") == "eu" and cfg.get_custom_property("x") is None
    cfg.authentication_type = "kerberos"
    with pytest.raises(ValueError):
        P.authentication_from(cfg)


def test_memory_and_local_registries(tmp_path):
    mem = P.MemoryRegistry()
    mem.add_model("tiny", _info("tiny"), b"abc")
    assert mem.count == 1 and mem.total_size == 3 and mem.can_handle("memory:zzz") and mem.can_handle("tiny") and not mem.can_handle("other")
    assert mem.model_exists("memory:tiny") and not mem.model_exists("tiny", "2.0.0") and mem.list_models() == ["tiny"]
    seen = []
    assert mem.download_model(mem.get_model_metadata("tiny"), seen.append) == b"abc" and seen == [1.0]
    with pytest.raises(E.ModelNotFoundError):
        mem.get_model_metadata("nope")
    assert mem.remove_model("tiny") and not mem.remove_model("tiny")

    (tmp_path / "a.bin").write_bytes(b"x" * 3000)
    (tmp_path / "b.pt").write_bytes(b"y" * 10)
    (tmp_path / "b.json").write_text(json.dumps({"name": "b", "architecture": "gpt", "config": {"n_layers": 2}, "version": "2.1.0", "tags": ["small"]}))
    os.makedirs(tmp_path / "c" / "3.0.0")
    (tmp_path / "c" / "3.0.0" / "c.bin").write_bytes(b"z")
    loc = P.LocalFileRegistry(str(tmp_path))
    assert loc.list_models() == ["a", "b", "c"]
    assert loc.can_handle("local:whatever") and loc.can_handle("a") and not loc.can_handle("zzz") and not loc.can_handle("../a")
    ia = loc.get_model_metadata("local:a")
    assert ia.file_size == 3000 and ia.framework_version == "BIN" and ia.source.endswith("a.bin")
    ib = loc.get_model_metadata("b")
    assert ib.version == "2.1.0" and ib.tags == ("small",) and ib.architecture == "gpt"
    assert loc.model_exists("b", "2.1.0") and not loc.model_exists("b", "9.9.9") and loc.model_exists("c", "3.0.0")
    prog = []
    assert loc.download_model(ia, prog.append) == b"x" * 3000 and prog[-1] == 1.0
    assert not loc.model_exists("../../etc/passwd")


def test_custom_registry_cache_expiry_and_retries():
    now = [0.0]
    naps = []

    class Flaky(P.CustomModelRegistry):
        registry_name = "flaky"
        priority = 10

        def __init__(self):
            super().__init__(P.PluginConfigurationBase(max_retries=3, retry_delay_milliseconds=250, cache_expiration_hours=1),
                             clock=lambda: now[0], sleep=naps.append)
            self.meta_calls = 0
            self.fail = 0

        def _fetch_metadata(self, name, version):
            self.meta_calls += 1
            if name == "gone":
                raise E.ModelNotFoundError(name)
            return _info(name, version or "1.0.0")

        def _fetch_model(self, metadata, progress):
            if self.fail > 0:
                self.fail -= 1
                raise ConnectionError("reset")
            return b"ok"

        def list_models(self):
            return ["x"]

    r = Flaky()
    assert r.can_handle("flaky/x") and r.can_handle("my-FLAKY-model") and not r.can_handle("other")
    r.get_model_metadata("x"); r.get_model_metadata("x")
    assert r.meta_calls == 1 and r.cached_entries == 1
    now[0] = 3601.0
    assert r.clean_expired_cache() == 1
    r.get_model_metadata("x")
    assert r.meta_calls == 2
    assert not r.model_exists("gone") and r.meta_calls == 3 and naps == []          # not-found is not retried
    r.fail = 2
    assert r.download_model(_info("x")) == b"ok" and naps == [0.25, 0.25] and len(r.log) == 2
    r.fail = 3
    with pytest.raises(E.DownloadFailedError) as ei:
        r.download_model(_info("x"))
    assert ei.value.retry_count == 3 and "reset" in str(ei.value)
    r.clear_cache()
    assert r.cached_entries == 0


def test_remote_registry_through_a_fake_transport():
    calls = []

    def transport(method, url, headers, timeout):
        calls.append((url, dict(headers)))
        if headers.get("X-API-Key") != "secret":
            return 401, {}, b""
        if url.endswith("/models"):
            return 200, {}, json.dumps({"models": ["r1", {"name": "r2"}]}).encode()
        if url.endswith("/models/r1"):
            return 200, {}, json.dumps({"version": "1.2.0", "task": "causal-lm", "unknown_field": 1}).encode()
        if url.endswith("/models/r1/1.2.0/download"):
            return 200, {}, b"weights"
        return 404, {}, b""

    cfg = P.AuthenticatedPluginConfiguration(authentication_type="apikey", api_key="secret", max_retries=1)
    r = P.RemoteRegistry("http://zoo.example/api/", cfg, transport=transport, sleep=lambda s: None)
    assert r.can_handle("remote:r1") and r.can_handle("http://zoo.example/api/models/r1") and not r.can_handle("r1")
    info = r.get_model_metadata("remote:r1")
    assert info.name == "r1" and info.version == "1.2.0" and info.architecture == "remote"
    assert r.download_model(info) == b"weights" and r.list_models() == ["r1", "r2"]
    assert not r.model_exists("r9")
    assert calls[0][0] == "http://zoo.example/api/models/r1" and calls[0][1]["X-API-Key"] == "secret"
    bad = P.RemoteRegistry("http://zoo.example/api", transport=transport)
    with pytest.raises(PermissionError):
        bad.get_model_metadata("r1")


def test_plugin_manager_priorities_extensions_and_fetch(tmp_path):
    (tmp_path / "shared.bin").write_bytes(b"from-disk")
    mem, loc = P.MemoryRegistry(), P.LocalFileRegistry(str(tmp_path))
    mem.add_model("shared", _info("shared"), b"from-memory")

    class Broken(P.ModelRegistryPlugin):
        registry_name, priority = "broken", 999

        def model_exists(self, n, v=None):
            raise RuntimeError("down")

        def can_handle(self, n):
            return False

    pm = P.PluginManager()
    for p in (loc, mem, Broken()):
        pm.register_plugin(p)
    with pytest.raises(ValueError):
        pm.register_plugin(P.MemoryRegistry())
    assert pm.list_plugins() == ["broken", "memory", "local"] and pm.plugin_count == 3
    assert pm.find_plugin("shared") is mem and pm.find_plugin("local:shared") is loc and pm.find_plugin("nobody") is None
    assert pm.get_best_source("shared") is mem and any("down" in m for m in pm.log)
    mem.remove_model("shared")
    assert pm.get_best_source("shared") is loc and pm.get_model_metadata("nothing") is None

    order = []

    class Decrypt(P.ModelZooExtension):
        extension_name, priority = "decrypt", 10

        def pre_download(self, m):
            order.append("decrypt.pre")

        def post_download(self, m, data):
            order.append("decrypt.post")
            return data.upper()

    class Audit(P.ModelZooExtension):
        extension_name, priority = "audit", 1

        def pre_download(self, m):
            order.append("audit.pre")

        def post_download(self, m, data):
            order.append("audit.post")
            raise RuntimeError("log full")

        def post_load(self, m):
            order.append("audit.loaded")

    pm.register_extension(Audit()); pm.register_extension(Decrypt())
    with pytest.raises(ValueError):
        pm.register_extension(Audit())
    info, data = pm.fetch("shared")
    assert data == b"FROM-DISK" and order == ["decrypt.pre", "audit.pre", "decrypt.post", "audit.post"]
    assert any("log full" in m for m in pm.log)
    pm.execute_pre_load_extensions(info); pm.execute_post_load_extensions(info)
    assert order[-1] == "audit.loaded"
    with pytest.raises(E.ModelNotFoundError):
        pm.fetch("nothing")
    assert pm.unregister_extension("audit") and not pm.unregister_extension("audit") and pm.extension_count == 1
    assert pm.unregister_plugin("broken") and not pm.unregister_plugin("broken")
    pm.clear_all()
    assert pm.plugin_count == 0 and pm.extension_count == 0


_PLUGIN_SRC = '''
from ml_framework_b200.modelzoo.plugins import (MemoryRegistry, PluginConfigurationBase, registry_plugin,
                                                registry_plugin_config)

@registry_plugin_config("{name}")
class Cfg(PluginConfigurationBase):
    pass

@registry_plugin("{name}", priority={prio})
class Mine(MemoryRegistry):
    def __init__(self, cfg):
        super().__init__()
        self.url = cfg.registry_url
'''


def test_discovery_from_directory_and_hot_reload(tmp_path):
    d = tmp_path / "plugins"
    d.mkdir()
    (d / "one.py").write_text(_PLUGIN_SRC.format(name="one", prio=5))
    (d / "_private.py").write_text("raise RuntimeError('never imported')")
    (d / "broken.py").write_text("import nonexistent_module_xyz")
    pm = P.PluginManager()
    disc = P.PluginDiscovery(pm, environ={"ONE_REGISTRY_URL": "http://one"})
    assert disc.load_plugins_from_directory(str(d)) == 1
    assert pm.list_plugins() == ["one"] and pm.get_plugin("one").url == "http://one" and pm.get_plugin("one").priority == 5
    assert len(disc.errors) == 1 and "nonexistent_module_xyz" in disc.errors[0]
    disc.enable_hot_reload(str(d))
    assert disc.get_watched_directories() == [str(d)] and disc.poll() == 0
    # a changed file replaces its plug-in, a new file adds one, a deleted file takes its plug-in away
    (d / "one.py").write_text(_PLUGIN_SRC.format(name="uno", prio=6))
    os.utime(d / "one.py", ns=(1, 1))
    (d / "two.py").write_text(_PLUGIN_SRC.format(name="two", prio=9))
    assert disc.poll() == 2 and pm.list_plugins() == ["two", "uno"]
    os.remove(d / "two.py")
    assert disc.poll() == 0 and pm.list_plugins() == ["uno"]
    disc.disable_all_hot_reload()
    assert disc.get_watched_directories() == [] and len(disc.get_loaded_modules()) >= 1
    with pytest.raises(FileNotFoundError):
        disc.load_plugins_from_directory(str(tmp_path / "absent"))
    # marked classes of an imported module
    import types
    mod = types.ModuleType("fake_plugin_module")

    @P.registry_plugin("inline", 3)
    class Inline(P.MemoryRegistry):
        pass
    mod.Inline = Inline
    assert disc.discover_plugins(mod) == 1 and disc.discover_plugins(mod) == 0 and pm.get_plugin("inline").priority == 3


def test_typed_errors_from_the_registry():
    reg = ZooRegistry()
    reg.register(_info("known", "1.0.0"))
    with pytest.raises(E.ModelNotFoundError) as e1:
        reg.get("unknown")
    assert e1.value.model_name == "unknown" and isinstance(e1.value, KeyError)
    with pytest.raises(E.VersionNotFoundError) as e2:
        reg.get("known", "3.0.0")
    assert e2.value.available == ["1.0.0"] and "available: 1.0.0" in str(e2.value)
    err = E.IncompatibleModelError("m", "1", "gpt", "llama")
    assert err.expected_architecture == "gpt" and "llama" in str(err)
    assert isinstance(E.ChecksumMismatchError("f", "a", "b"), IOError) and isinstance(E.DownloadTimeoutError("u", 10), TimeoutError)
    assert E.DeserializationError("f.bin", "bad magic").file_path == "f.bin"
