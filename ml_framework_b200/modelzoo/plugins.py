"""Registry plug-ins and load-flow extensions of the model zoo.

Reference: src/ModelZoo/Plugins — IModelRegistryPlugin.cs:9-58, IModelZooExtension.cs:10-77,
IRegistryAuthentication.cs:9-112, PluginConfiguration.cs:11-185, CustomModelRegistry.cs:17-285,
PluginManager.cs:12-406, PluginDiscovery.cs:14-315, RegistryPluginAttribute.cs:7-57,
BuiltIn/MemoryRegistry.cs:14-211, BuiltIn/LocalFileRegistry.cs:13-161,
BuiltIn/RemoteRegistry.cs:15-259.

A registry plug-in answers four questions about a model name (does it exist, what is its
card, give me its bytes, what do you have) and says whether a name is its business at all;
the manager asks the plug-ins in priority order. Extensions hook the four points of a load
(before / after download, before / after load). Discovery finds plug-in classes marked with
``@registry_plugin`` in modules or in a directory of ``*.py`` files, and reloads files of a
watched directory when their modification time changes. Network access goes through an
injectable transport, so everything here is testable without a network.
"""
from __future__ import annotations

import base64
import dataclasses
import fnmatch
import importlib.util
import json
import os
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple, Type

from .errors import DownloadFailedError, ModelNotFoundError
from .zoo import ModelInfo

__all__ = [
    "ApiKeyAuthentication", "TokenAuthentication", "BasicAuthentication", "CustomAuthentication",
    "PluginConfigurationBase", "AuthenticatedPluginConfiguration", "PluginConfigurationLoader",
    "authentication_from", "ModelRegistryPlugin", "CustomModelRegistry", "MemoryRegistry",
    "LocalFileRegistry", "RemoteRegistry", "ModelZooExtension", "PluginManager", "registry_plugin",
    "registry_plugin_config", "PluginDiscovery",
]

Progress = Optional[Callable[[float], None]]
Transport = Callable[[str, str, Dict[str, str], float], Tuple[int, Dict[str, str], bytes]]


# ------------------------------------------------------------------ authentication
class ApiKeyAuthentication:
    scheme = "ApiKey"

    def __init__(self, api_key: str, header_name: str = "X-API-Key"):
        if not api_key:
            raise ValueError("the API key cannot be empty")
        self._key, self.header_name = api_key, header_name

    def authenticate(self, headers: Dict[str, str]) -> None:
        headers[self.header_name] = self._key


class TokenAuthentication:
    def __init__(self, token: str, token_type: str = "Bearer"):
        if not token:
            raise ValueError("the token cannot be empty")
        self._token, self.scheme = token, token_type

    def authenticate(self, headers: Dict[str, str]) -> None:
        headers["Authorization"] = f"{self.scheme} {self._token}"


class BasicAuthentication:
    scheme = "Basic"

    def __init__(self, username: str, password: str):
        if not username:
            raise ValueError("the user name cannot be empty")
        self._cred = base64.b64encode(f"{username}:{password}".encode()).decode()

    def authenticate(self, headers: Dict[str, str]) -> None:
        headers["Authorization"] = f"Basic {self._cred}"


class CustomAuthentication:
    def __init__(self, action: Callable[[Dict[str, str]], None], scheme: str = "Custom"):
        self._action, self.scheme = action, scheme

    def authenticate(self, headers: Dict[str, str]) -> None:
        self._action(headers)


# ------------------------------------------------------------------ configuration
@dataclass
class PluginConfigurationBase:
    registry_url: str = ""
    enable_caching: bool = True
    cache_directory: str = ""
    cache_expiration_hours: int = 24
    http_timeout_seconds: int = 300
    max_retries: int = 3
    retry_delay_milliseconds: int = 1000
    custom_properties: Dict[str, str] = field(default_factory=dict)

    def get_custom_property(self, key: str) -> Optional[str]:
        return self.custom_properties.get(key)

    def set_custom_property(self, key: str, value: str) -> None:
        self.custom_properties[key] = value


@dataclass
class AuthenticatedPluginConfiguration(PluginConfigurationBase):
    authentication_type: str = ""          # "" | apikey | token | basic
    api_key: str = ""
    api_key_header_name: str = "X-API-Key"
    token: str = ""
    token_type: str = "Bearer"
    username: str = ""
    password: str = ""
    credentials_encrypted: bool = False


class PluginConfigurationLoader:
    """Fills a configuration from ``<PREFIX>_<FIELD>`` environment variables
    (PluginConfiguration.cs:124-183); unparsable numbers and booleans leave the default."""

    @staticmethod
    def load_value(name: str, environ: Optional[Dict[str, str]] = None) -> str:
        return (os.environ if environ is None else environ).get(name, "")

    @classmethod
    def load_from_environment(cls, config_type: Type[PluginConfigurationBase], prefix: str,
                              environ: Optional[Dict[str, str]] = None) -> PluginConfigurationBase:
        cfg = config_type()
        for f in dataclasses.fields(cfg):
            raw = cls.load_value(f"{prefix}_{f.name.upper()}", environ)
            if not raw:
                continue
            cur = getattr(cfg, f.name)
            if isinstance(cur, bool):
                if raw.strip().lower() in ("true", "false"):
                    setattr(cfg, f.name, raw.strip().lower() == "true")
            elif isinstance(cur, int):
                try:
                    setattr(cfg, f.name, int(raw))
                except ValueError:
                    pass
            elif isinstance(cur, str):
                setattr(cfg, f.name, raw)
        return cfg


def authentication_from(cfg: PluginConfigurationBase):
    """The authentication object an ``AuthenticatedPluginConfiguration`` describes, or ``None``."""
    kind = getattr(cfg, "authentication_type", "").lower()
    if not kind:
        return None
    if getattr(cfg, "credentials_encrypted", False):
        raise ValueError("encrypted credentials need a CustomAuthentication that decrypts them")
    if kind == "apikey":
        return ApiKeyAuthentication(cfg.api_key, cfg.api_key_header_name)
    if kind in ("token", "bearer"):
        return TokenAuthentication(cfg.token, cfg.token_type)
    if kind == "basic":
        return BasicAuthentication(cfg.username, cfg.password)
    raise ValueError(f"unknown authentication type {cfg.authentication_type!r}")


# ------------------------------------------------------------------ plug-in interface
class ModelRegistryPlugin:
    """Interface of a registry plug-in. Higher ``priority`` is asked first."""

    registry_name: str = "plugin"
    priority: int = 0

    def get_model_metadata(self, model_name: str, version: Optional[str] = None) -> ModelInfo:
        raise NotImplementedError

    def download_model(self, metadata: ModelInfo, progress: Progress = None) -> bytes:
        raise NotImplementedError

    def model_exists(self, model_name: str, version: Optional[str] = None) -> bool:
        raise NotImplementedError

    def list_models(self) -> List[str]:
        raise NotImplementedError

    def can_handle(self, model_name: str) -> bool:
        raise NotImplementedError


class CustomModelRegistry(ModelRegistryPlugin):
    """Base with a metadata cache that expires and a retry loop around the two fetches
    (CustomModelRegistry.cs:17-285). Subclasses give ``_fetch_metadata`` and ``_fetch_model``."""

    def __init__(self, configuration: Optional[PluginConfigurationBase] = None, clock: Callable[[], float] = time.time,
                 sleep: Callable[[float], None] = time.sleep):
        self.configuration = configuration or PluginConfigurationBase()
        self._clock, self._sleep = clock, sleep
        self._cache: Dict[str, Tuple[float, ModelInfo]] = {}
        self._lock = threading.RLock()
        self.log: List[str] = []

    # subclasses
    def _fetch_metadata(self, model_name: str, version: Optional[str]) -> ModelInfo:
        raise NotImplementedError

    def _fetch_model(self, metadata: ModelInfo, progress: Progress) -> bytes:
        raise NotImplementedError

    @staticmethod
    def _cache_key(model_name: str, version: Optional[str]) -> str:
        return f"{model_name}:{version}" if version else model_name

    def _retry(self, what: str, fn):
        last: Optional[BaseException] = None
        tries = max(1, self.configuration.max_retries)
        for attempt in range(tries):
            try:
                return fn()
            except (ModelNotFoundError, FileNotFoundError, PermissionError):
                raise                                    # asking again cannot help
            except Exception as e:                       # noqa: BLE001 - any transport error is retried
                last = e
                self.log.append(f"[{self.registry_name}] {what}: attempt {attempt + 1}/{tries} failed: {e}")
                if attempt + 1 < tries:
                    self._sleep(self.configuration.retry_delay_milliseconds / 1000.0)
        raise DownloadFailedError([self.configuration.registry_url or self.registry_name], tries,
                                  f"{self.registry_name}: {what} failed after {tries} attempts: {last}") from last

    def get_model_metadata(self, model_name: str, version: Optional[str] = None) -> ModelInfo:
        if not model_name:
            raise ValueError("the model name cannot be empty")
        key = self._cache_key(model_name, version)
        ttl = self.configuration.cache_expiration_hours * 3600.0
        with self._lock:
            hit = self._cache.get(key)
            if self.configuration.enable_caching and hit and self._clock() - hit[0] < ttl:
                return hit[1]
        info = self._retry(f"metadata of {key}", lambda: self._fetch_metadata(model_name, version))
        if self.configuration.enable_caching:
            with self._lock:
                self._cache[key] = (self._clock(), info)
        return info

    def download_model(self, metadata: ModelInfo, progress: Progress = None) -> bytes:
        return self._retry(f"download of {metadata.name}", lambda: self._fetch_model(metadata, progress))

    def model_exists(self, model_name: str, version: Optional[str] = None) -> bool:
        try:
            self.get_model_metadata(model_name, version)
            return True
        except (KeyError, FileNotFoundError, DownloadFailedError):
            return False

    def can_handle(self, model_name: str) -> bool:
        if not model_name:
            return False
        n, r = model_name.lower(), self.registry_name.lower()
        return n.startswith(r + "/") or r in n

    def clear_cache(self) -> None:
        with self._lock:
            self._cache.clear()

    def clean_expired_cache(self) -> int:
        ttl = self.configuration.cache_expiration_hours * 3600.0
        with self._lock:
            dead = [k for k, (t, _) in self._cache.items() if self._clock() - t >= ttl]
            for k in dead:
                del self._cache[k]
        return len(dead)

    @property
    def cached_entries(self) -> int:
        return len(self._cache)


# ------------------------------------------------------------------ built-in registries
class MemoryRegistry(ModelRegistryPlugin):
    """Models held in memory: for tests and for models made in this process (priority 200)."""

    registry_name = "memory"
    priority = 200

    def __init__(self):
        self._m: Dict[str, Tuple[ModelInfo, bytes]] = {}
        self._lock = threading.Lock()

    def add_model(self, model_name: str, metadata: ModelInfo, data: bytes) -> None:
        if not model_name:
            raise ValueError("the model name cannot be empty")
        if metadata is None or data is None:
            raise ValueError("metadata and data are required")
        with self._lock:
            self._m[model_name] = (metadata, bytes(data))

    def remove_model(self, model_name: str) -> bool:
        with self._lock:
            return self._m.pop(model_name, None) is not None

    def clear(self) -> None:
        with self._lock:
            self._m.clear()

    @staticmethod
    def _bare(model_name: str) -> str:
        return model_name[7:] if model_name.lower().startswith("memory:") else model_name

    def get_model_metadata(self, model_name, version=None) -> ModelInfo:
        with self._lock:
            hit = self._m.get(self._bare(model_name))
        if hit is None or (version is not None and hit[0].version != version):
            raise ModelNotFoundError(model_name)
        return hit[0]

    def download_model(self, metadata: ModelInfo, progress: Progress = None) -> bytes:
        with self._lock:
            hit = self._m.get(metadata.name)
        if hit is None:
            raise ModelNotFoundError(metadata.name)
        if progress:
            progress(1.0)
        return hit[1]

    def model_exists(self, model_name, version=None) -> bool:
        with self._lock:
            hit = self._m.get(self._bare(model_name))
        return hit is not None and (version is None or hit[0].version == version)

    def list_models(self) -> List[str]:
        with self._lock:
            return sorted(self._m)

    def can_handle(self, model_name: str) -> bool:
        return bool(model_name) and (model_name.lower().startswith("memory:") or self.model_exists(model_name))

    @property
    def count(self) -> int:
        return len(self._m)

    @property
    def total_size(self) -> int:
        with self._lock:
            return sum(len(d) for _, d in self._m.values())


_EXTENSIONS = (".bin", ".pt", ".pth", ".safetensors", ".mlfw", ".onnx", ".pb", ".h5", "")


class LocalFileRegistry(CustomModelRegistry):
    """Weight files under one directory; ``local:<name>`` or a bare name that exists there
    (priority 100). A ``<name>.json`` card beside the file supplies the metadata; without one the
    card is made from the file's facts."""

    registry_name = "local"
    priority = 100

    def __init__(self, base_directory: str, configuration: Optional[PluginConfigurationBase] = None, **kw):
        if not base_directory:
            raise ValueError("the base directory cannot be empty")
        super().__init__(configuration, **kw)
        os.makedirs(base_directory, exist_ok=True)
        self.base_directory = os.path.abspath(base_directory)

    def _path(self, model_name: str, version: Optional[str] = None) -> Optional[str]:
        name = model_name[6:] if model_name.lower().startswith("local:") else model_name
        if os.path.isabs(name) or ".." in name.replace("\\", "/").split("/"):
            return None                                   # never leave the base directory
        stems = ([os.path.join(name, version, name), os.path.join(version, name), f"{name}-{version}"] if version else []) + [name]
        for stem in stems:
            for ext in _EXTENSIONS:
                p = os.path.join(self.base_directory, stem + ext)
                if os.path.isfile(p):
                    return p
        return None

    def _fetch_metadata(self, model_name, version) -> ModelInfo:
        p = self._path(model_name, version)
        if p is None:
            raise ModelNotFoundError(model_name)
        bare = os.path.splitext(os.path.basename(p))[0]
        card = os.path.splitext(p)[0] + ".json"
        st = os.stat(p)
        if os.path.isfile(card):
            with open(card) as f:
                d = json.load(f)
            d["tags"] = tuple(d.get("tags", ()))
            d.setdefault("name", bare)
            d.setdefault("architecture", "local")
            d.setdefault("config", {})
            info = ModelInfo(**d)
            if version is not None and info.version != version:
                raise ModelNotFoundError(model_name)
        else:
            info = ModelInfo(name=bare, architecture="local", config={}, version=version or "1.0.0",
                             description=f"model file {os.path.basename(p)} of the local registry",
                             framework_version=os.path.splitext(p)[1].lstrip(".").upper())
        info.source, info.file_size = p, st.st_size
        return info

    def _fetch_model(self, metadata: ModelInfo, progress: Progress) -> bytes:
        p = metadata.source
        if not p or not os.path.isfile(p):
            raise FileNotFoundError(f"model file not found: {p!r}")
        total, chunks, done = max(1, os.path.getsize(p)), [], 0
        with open(p, "rb") as f:
            for c in iter(lambda: f.read(1 << 20), b""):
                chunks.append(c)
                done += len(c)
                if progress:
                    progress(done / total)
        return b"".join(chunks)

    def list_models(self) -> List[str]:
        out = set()
        for dp, _, fns in os.walk(self.base_directory):
            for fn in fns:
                if not fn.endswith(".json"):
                    out.add(os.path.splitext(fn)[0])
        return sorted(out)

    def can_handle(self, model_name: str) -> bool:
        return bool(model_name) and (model_name.lower().startswith("local:") or self._path(model_name) is not None)


class RemoteRegistry(CustomModelRegistry):
    """HTTP registry: ``GET <base>/models/<name>[/<version>]`` gives the card as JSON,
    ``GET <base>/models/<name>/<version>/download`` the bytes, ``GET <base>/models`` the names
    (priority 50). Names ``remote:<name>`` or ``<base-url>/...`` are its business."""

    registry_name = "remote"
    priority = 50

    def __init__(self, base_url: str, configuration: Optional[AuthenticatedPluginConfiguration] = None,
                 transport: Optional[Transport] = None, authentication=None, **kw):
        if not base_url:
            raise ValueError("the base URL cannot be empty")
        cfg = configuration or AuthenticatedPluginConfiguration()
        cfg.registry_url = cfg.registry_url or base_url
        super().__init__(cfg, **kw)
        self.base_url = base_url.rstrip("/")
        self.authentication = authentication or authentication_from(cfg)
        if transport is None:
            from .hubs import urllib_transport
            transport = urllib_transport
        self._transport = transport

    def _get(self, url: str) -> bytes:
        headers: Dict[str, str] = {"Accept": "application/json, application/octet-stream"}
        if self.authentication is not None:
            self.authentication.authenticate(headers)
        status, _, body = self._transport("GET", url, headers, float(self.configuration.http_timeout_seconds))
        if status == 404:
            raise ModelNotFoundError(url)
        if status in (401, 403):
            raise PermissionError(f"{self.registry_name}: HTTP {status} for {url}")
        if status >= 400:
            raise ConnectionError(f"{self.registry_name}: HTTP {status} for {url}")
        return body

    @staticmethod
    def _bare(model_name: str) -> str:
        return model_name[7:] if model_name.lower().startswith("remote:") else model_name

    def _fetch_metadata(self, model_name, version) -> ModelInfo:
        name = self._bare(model_name)
        url = f"{self.base_url}/models/{name}" + (f"/{version}" if version else "")
        try:
            d = json.loads(self._get(url).decode())
        except ModelNotFoundError:
            raise ModelNotFoundError(model_name) from None
        d["tags"] = tuple(d.get("tags", ()))
        d.setdefault("name", name)
        d.setdefault("architecture", "remote")
        d.setdefault("config", {})
        known = {f.name for f in dataclasses.fields(ModelInfo)}
        return ModelInfo(**{k: v for k, v in d.items() if k in known})

    def _fetch_model(self, metadata: ModelInfo, progress: Progress) -> bytes:
        url = metadata.source if metadata.source and "://" in metadata.source else \
            f"{self.base_url}/models/{metadata.name}/{metadata.version}/download"
        body = self._get(url)
        if progress:
            progress(1.0)
        return body

    def list_models(self) -> List[str]:
        data = json.loads(self._retry("model list", lambda: self._get(f"{self.base_url}/models")).decode())
        return [m if isinstance(m, str) else m.get("name", "") for m in (data.get("models", []) if isinstance(data, dict) else data)]

    def can_handle(self, model_name: str) -> bool:
        if not model_name:
            return False
        n = model_name.lower()
        return n.startswith("remote:") or n.startswith(self.base_url.lower())


# ------------------------------------------------------------------ extensions
class ModelZooExtension:
    """Hooks round a model load; override what you need (IModelZooExtension.cs:10-77)."""

    extension_name: str = "extension"
    priority: int = 0

    def pre_download(self, metadata: ModelInfo) -> None:
        pass

    def post_download(self, metadata: ModelInfo, data: bytes) -> bytes:
        return data

    def pre_load(self, metadata: ModelInfo) -> None:
        pass

    def post_load(self, metadata: ModelInfo) -> None:
        pass


class PluginManager:
    """Keeps plug-ins by name and extensions by priority (PluginManager.cs:12-406)."""

    def __init__(self):
        self._plugins: Dict[str, ModelRegistryPlugin] = {}
        self._extensions: List[ModelZooExtension] = []
        self._lock = threading.RLock()
        self.log: List[str] = []

    # ---- plug-ins
    def register_plugin(self, plugin: ModelRegistryPlugin) -> None:
        if plugin is None or not getattr(plugin, "registry_name", ""):
            raise ValueError("a plug-in needs a registry name")
        with self._lock:
            if plugin.registry_name in self._plugins:
                raise ValueError(f"a plug-in named {plugin.registry_name!r} is already registered")
            self._plugins[plugin.registry_name] = plugin

    def unregister_plugin(self, registry_name: str) -> bool:
        with self._lock:
            p = self._plugins.pop(registry_name, None)
        if p is not None and hasattr(p, "close"):
            p.close()
        return p is not None

    def get_plugin(self, registry_name: str) -> Optional[ModelRegistryPlugin]:
        return self._plugins.get(registry_name)

    def list_plugins(self) -> List[str]:
        return [p.registry_name for p in self.get_all_plugins()]

    def get_all_plugins(self) -> List[ModelRegistryPlugin]:
        with self._lock:
            return sorted(self._plugins.values(), key=lambda p: -p.priority)

    def find_plugin(self, model_name: str) -> Optional[ModelRegistryPlugin]:
        """The highest-priority plug-in that claims the name."""
        if not model_name:
            raise ValueError("the model name cannot be empty")
        return next((p for p in self.get_all_plugins() if p.can_handle(model_name)), None)

    def get_best_source(self, model_name: str, version: Optional[str] = None) -> Optional[ModelRegistryPlugin]:
        """The highest-priority plug-in that has the model; a plug-in that fails is passed over."""
        if not model_name:
            raise ValueError("the model name cannot be empty")
        for p in self.get_all_plugins():
            try:
                if p.model_exists(model_name, version):
                    return p
            except Exception as e:                       # noqa: BLE001 - one broken registry must not hide the others
                self.log.append(f"registry {p.registry_name}: {e}")
        return None

    def get_model_metadata(self, model_name: str, version: Optional[str] = None) -> Optional[ModelInfo]:
        p = self.get_best_source(model_name, version)
        return p.get_model_metadata(model_name, version) if p is not None else None

    def fetch(self, model_name: str, version: Optional[str] = None, progress: Progress = None) -> Tuple[ModelInfo, bytes]:
        """Card and bytes from the best source, with the download hooks run round the transfer."""
        p = self.get_best_source(model_name, version)
        if p is None:
            raise ModelNotFoundError(model_name)
        info = p.get_model_metadata(model_name, version)
        self.execute_pre_download_extensions(info)
        data = p.download_model(info, progress)
        return info, self.execute_post_download_extensions(info, data)

    # ---- extensions
    def register_extension(self, ext: ModelZooExtension) -> None:
        if ext is None:
            raise ValueError("the extension is required")
        with self._lock:
            if any(e.extension_name == ext.extension_name for e in self._extensions):
                raise ValueError(f"an extension named {ext.extension_name!r} is already registered")
            self._extensions.append(ext)
            self._extensions.sort(key=lambda e: -e.priority)

    def unregister_extension(self, extension_name: str) -> bool:
        with self._lock:
            n = len(self._extensions)
            self._extensions = [e for e in self._extensions if e.extension_name != extension_name]
            return len(self._extensions) < n

    def get_all_extensions(self) -> List[ModelZooExtension]:
        with self._lock:
            return list(self._extensions)

    def _each(self, hook: str, metadata: ModelInfo):
        for e in self.get_all_extensions():
            try:
                getattr(e, hook)(metadata)
            except Exception as err:                     # noqa: BLE001 - a failing hook is recorded, the load goes on
                self.log.append(f"extension {e.extension_name}.{hook}: {err}")

    def execute_pre_download_extensions(self, metadata: ModelInfo) -> None:
        self._each("pre_download", metadata)

    def execute_post_download_extensions(self, metadata: ModelInfo, data: bytes) -> bytes:
        for e in self.get_all_extensions():
            try:
                out = e.post_download(metadata, data)
                data = data if out is None else out
            except Exception as err:                     # noqa: BLE001
                self.log.append(f"extension {e.extension_name}.post_download: {err}")
        return data

    def execute_pre_load_extensions(self, metadata: ModelInfo) -> None:
        self._each("pre_load", metadata)

    def execute_post_load_extensions(self, metadata: ModelInfo) -> None:
        self._each("post_load", metadata)

    @property
    def plugin_count(self) -> int:
        return len(self._plugins)

    @property
    def extension_count(self) -> int:
        return len(self._extensions)

    def clear_all(self) -> None:
        for name in list(self._plugins):
            self.unregister_plugin(name)
        with self._lock:
            self._extensions.clear()


# ------------------------------------------------------------------ discovery
def registry_plugin(name: str, priority: int = 0):
    """Class decorator that marks a plug-in for discovery and sets its name and priority."""
    if not name:
        raise ValueError("a plug-in needs a name")

    def mark(cls):
        cls.registry_name, cls.priority = name, priority
        cls.__registry_plugin__ = True
        return cls
    return mark


def registry_plugin_config(registry_name: str):
    """Class decorator that ties a configuration class to a plug-in name; discovery builds the
    configuration from ``<NAME>_*`` environment variables and passes it to the plug-in."""
    def mark(cls):
        cls.__registry_plugin_config__ = registry_name
        return cls
    return mark


class PluginDiscovery:
    """Finds marked plug-in classes in modules and in directories of ``*.py`` files, and reloads a
    watched directory's files when they change (PluginDiscovery.cs:14-315). Watching is by
    polling: call ``poll()`` (a background thread does when ``interval_s`` is given)."""

    def __init__(self, plugin_manager: PluginManager, environ: Optional[Dict[str, str]] = None):
        if plugin_manager is None:
            raise ValueError("the plug-in manager is required")
        self.manager = plugin_manager
        self._environ = environ
        self._modules: Dict[str, object] = {}                 # path or module name -> module
        self._from_file: Dict[str, List[str]] = {}            # path -> plug-in names it registered
        self._watched: Dict[str, Dict[str, float]] = {}       # directory -> {file: mtime}
        self._threads: Dict[str, Tuple[threading.Thread, threading.Event]] = {}
        self.errors: List[str] = []

    def discover_plugins(self, module) -> int:
        """Registers every marked class of ``module`` that is not yet registered; returns the count."""
        configs = {getattr(c, "__registry_plugin_config__"): c for c in vars(module).values()
                   if isinstance(c, type) and hasattr(c, "__registry_plugin_config__")}
        n = 0
        for cls in list(vars(module).values()):
            if not (isinstance(cls, type) and cls.__dict__.get("__registry_plugin__")):
                continue
            if self.manager.get_plugin(cls.registry_name) is not None:
                continue
            try:
                if cls.registry_name in configs:
                    cfg = PluginConfigurationLoader.load_from_environment(
                        configs[cls.registry_name], cls.registry_name.upper(), self._environ)
                    plugin = cls(cfg)
                else:
                    plugin = cls()
                self.manager.register_plugin(plugin)
                n += 1
            except Exception as e:                       # noqa: BLE001 - one bad plug-in does not stop discovery
                self.errors.append(f"{cls.__name__}: {e}")
        self._modules.setdefault(getattr(module, "__name__", str(id(module))), module)
        return n

    def discover_all_plugins(self) -> int:
        """Every module already imported whose name mentions ``plugin``."""
        return sum(self.discover_plugins(m) for name, m in list(sys.modules.items())
                   if m is not None and "plugin" in name.lower() and name != __name__)

    def load_plugin_file(self, path: str) -> int:
        path = os.path.abspath(path)
        if not os.path.isfile(path):
            raise FileNotFoundError(path)
        for name in self._from_file.pop(path, []):           # a reload replaces what the file gave before
            self.manager.unregister_plugin(name)
        mod_name = f"_mlf_zoo_plugin_{abs(hash(path)):x}"
        spec = importlib.util.spec_from_file_location(mod_name, path)
        module = importlib.util.module_from_spec(spec)
        try:
            spec.loader.exec_module(module)
        except Exception as e:                           # noqa: BLE001
            self.errors.append(f"{path}: {e}")
            return 0
        before = set(self.manager.list_plugins())
        n = self.discover_plugins(module)
        self._modules[path] = module
        self._from_file[path] = [p for p in self.manager.list_plugins() if p not in before]
        return n

    def load_plugins_from_directory(self, directory: str, search_pattern: str = "*.py") -> int:
        if not os.path.isdir(directory):
            raise FileNotFoundError(directory)
        return sum(self.load_plugin_file(os.path.join(directory, fn)) for fn in sorted(os.listdir(directory))
                   if fnmatch.fnmatch(fn, search_pattern) and not fn.startswith("_"))

    # ---- hot reload
    def _scan(self, directory: str) -> Dict[str, float]:
        return {os.path.join(directory, fn): os.stat(os.path.join(directory, fn)).st_mtime_ns
                for fn in os.listdir(directory) if fn.endswith(".py") and not fn.startswith("_")}

    def enable_hot_reload(self, directory: str, interval_s: Optional[float] = None) -> None:
        directory = os.path.abspath(directory)
        if not os.path.isdir(directory):
            raise FileNotFoundError(directory)
        self._watched[directory] = self._scan(directory)
        if interval_s is not None and directory not in self._threads:
            stop = threading.Event()

            def loop():
                while not stop.wait(interval_s):
                    self.poll()
            t = threading.Thread(target=loop, name="mlf-plugin-watch", daemon=True)
            self._threads[directory] = (t, stop)
            t.start()

    def poll(self) -> int:
        """Loads new and changed files of the watched directories, drops the plug-ins of deleted
        files; returns how many files were (re)loaded."""
        n = 0
        for d, seen in list(self._watched.items()):
            if not os.path.isdir(d):
                continue
            now = self._scan(d)
            for path, m in now.items():
                if seen.get(path) != m:
                    self.load_plugin_file(path)
                    n += 1
            for path in set(seen) - set(now):
                for name in self._from_file.pop(path, []):
                    self.manager.unregister_plugin(name)
                self._modules.pop(path, None)
            self._watched[d] = now
        return n

    def disable_hot_reload(self, directory: str) -> None:
        directory = os.path.abspath(directory)
        self._watched.pop(directory, None)
        t = self._threads.pop(directory, None)
        if t is not None:
            t[1].set()
            t[0].join(timeout=5)

    def disable_all_hot_reload(self) -> None:
        for d in list(self._watched):
            self.disable_hot_reload(d)

    def get_loaded_modules(self) -> List[object]:
        return list(self._modules.values())

    def get_watched_directories(self) -> List[str]:
        return sorted(self._watched)
