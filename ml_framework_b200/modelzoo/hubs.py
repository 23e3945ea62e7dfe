"""External model hubs: Hugging Face, TensorFlow Hub and the ONNX model zoo behind one interface, a registry that
routes model ids to hubs, id parsing and authentication.

Interface and behaviour follow the reference (src/ModelZoo/ExternalHubs/IModelHub.cs: hub name, authentication,
configuration, ``get_model_metadata``, ``download_model``, ``model_exists``, ``list_models``, ``can_handle``;
ModelIdParser.cs:72-160 for ``hub:<hub>/<model>[/<version>[/<variant>]]`` and ``hub:<registry>:<path>`` ids;
HubRegistry.cs:25-200; HubConfiguration.cs for time-outs, retries, mirrors and base URLs; HuggingFaceHub.cs:62-210,
TensorFlowHub.cs:68-140, ONNXHub.cs:73-205 for the URL schemes). All traffic goes through a ``transport`` callable
``(method, url, headers, timeout) -> (status, headers, body bytes)``; the default one uses ``urllib``, tests and
air-gapped sites pass their own (a directory mirror, a cache, a fake).
"""
from __future__ import annotations

import json
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

Transport = Callable[[str, str, Dict[str, str], float], Tuple[int, Dict[str, str], bytes]]


# ------------------------------------------------------------------ ids
@dataclass
class ModelIdComponents:
    hub_name: Optional[str] = None
    model_name: str = ""
    version: Optional[str] = None
    variant: Optional[str] = None

    @property
    def is_local(self) -> bool:
        return self.hub_name is None

    @property
    def full_id(self) -> str:
        if self.is_local:
            return self.model_name
        parts = [self.model_name] + [p for p in (self.version, self.variant) if p]
        return f"hub:{self.hub_name}/" + "/".join(parts)


def parse_model_id(model_id: str) -> ModelIdComponents:
    if not model_id or not model_id.strip():
        raise ValueError("model id cannot be empty")
    c = ModelIdComponents()
    if not model_id.startswith("hub:"):
        c.model_name = model_id
        return c
    rest = model_id[4:]
    if ":" in rest:
        c.hub_name, rest = rest.split(":", 1)
    else:
        if "/" not in rest:
            raise ValueError(f"invalid model id {model_id!r}: expected 'hub:huggingface/bert-base-uncased'")
        c.hub_name, rest = rest.split("/", 1)
    parts = rest.split("/")
    if not parts or not parts[0]:
        raise ValueError(f"invalid model id {model_id!r}: a model name is required")
    c.model_name = parts[0]
    c.version = parts[1] if len(parts) > 1 else None
    c.variant = parts[2] if len(parts) > 2 else None
    return c


def is_local_model(model_id: str) -> bool:
    return not model_id.startswith("hub:")


# ------------------------------------------------------------------ authentication / configuration
class AnonymousAuth:
    auth_type = "anonymous"

    def get_auth_header(self) -> Tuple[str, str]:
        return "", ""

    def is_valid(self) -> bool:
        return True


class ApiKeyAuth:
    auth_type = "api_key"

    def __init__(self, key: str, header_name: str = "X-API-Key"):
        self.key, self.header_name = key, header_name

    def get_auth_header(self):
        return self.header_name, self.key

    def is_valid(self) -> bool:
        return bool(self.key)


class TokenAuth:
    auth_type = "token"

    def __init__(self, token: str):
        self.token = token

    def get_auth_header(self):
        return "Authorization", f"Bearer {self.token}"

    def is_valid(self) -> bool:
        return bool(self.token)


@dataclass
class HubConfiguration:
    timeout_seconds: int = 300
    max_retries: int = 3
    retry_delay_seconds: float = 5.0
    verify_ssl: bool = True
    custom_headers: Dict[str, str] = field(default_factory=dict)

    def is_valid(self) -> bool:
        return self.timeout_seconds > 0 and self.max_retries >= 0 and self.retry_delay_seconds >= 0


@dataclass
class HuggingFaceHubConfiguration(HubConfiguration):
    api_token: Optional[str] = None
    default_repository: str = "models"
    base_url: str = "https://huggingface.co"
    use_mirror: bool = False
    mirror_url: Optional[str] = None

    @property
    def effective_base_url(self) -> str:
        return self.mirror_url if self.use_mirror and self.mirror_url else self.base_url

    def is_valid(self) -> bool:
        return super().is_valid() and bool(self.effective_base_url)


@dataclass
class TensorFlowHubConfiguration(HubConfiguration):
    base_url: str = "https://tfhub.dev"
    use_compression: bool = True
    compression_format: str = "gzip"
    preferred_format: str = "saved_model"

    def is_valid(self) -> bool:
        return super().is_valid() and bool(self.base_url)


@dataclass
class ONNXHubConfiguration(HubConfiguration):
    base_url: str = "https://github.com/onnx/models"
    raw_content_url: str = "https://raw.githubusercontent.com/onnx/models/main"
    mirror_urls: List[str] = field(default_factory=list)
    prefer_mirrors: bool = False
    default_version: str = "latest"

    def is_valid(self) -> bool:
        return super().is_valid() and bool(self.raw_content_url)


@dataclass
class HubModelMetadata:
    model_name: str
    description: str = ""
    framework: str = "pytorch"
    architecture: str = "unknown"
    custom: Dict[str, str] = field(default_factory=dict)


class HubError(RuntimeError):
    pass


def urllib_transport(method: str, url: str, headers: Dict[str, str], timeout: float):
    req = urllib.request.Request(url, method=method, headers=headers)
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.status, dict(r.headers), r.read()
    except urllib.error.HTTPError as e:
        return e.code, dict(e.headers or {}), b""


# ------------------------------------------------------------------ hubs
class ModelHub:
    hub_name = "hub"
    aliases: Tuple[str, ...] = ()

    def __init__(self, configuration: HubConfiguration, authentication=None, transport: Optional[Transport] = None, sleep=time.sleep):
        if not configuration.is_valid():
            raise ValueError(f"invalid configuration for hub {self.hub_name!r}")
        self.configuration, self.authentication = configuration, authentication
        self.transport, self._sleep = transport or urllib_transport, sleep

    def _headers(self) -> Dict[str, str]:
        h = dict(self.configuration.custom_headers)
        a = self.authentication
        if a is not None and a.is_valid() and a.auth_type != "anonymous":
            k, v = a.get_auth_header()
            if k:
                h[k] = v
        return h

    def _request(self, method: str, url: str) -> Tuple[int, Dict[str, str], bytes]:
        """Transport errors and 5xx answers are retried ``max_retries`` times with ``retry_delay_seconds`` between."""
        last: Optional[Exception] = None
        for attempt in range(self.configuration.max_retries + 1):
            try:
                status, hdr, body = self.transport(method, url, self._headers(), float(self.configuration.timeout_seconds))
                if status < 500:
                    return status, hdr, body
                last = HubError(f"{method} {url}: HTTP {status}")
            except (OSError, TimeoutError) as e:
                last = e
            if attempt < self.configuration.max_retries:
                self._sleep(self.configuration.retry_delay_seconds)
        raise HubError(f"{method} {url} failed after {self.configuration.max_retries + 1} attempts: {last}")

    def can_handle(self, model_id: str) -> bool:
        try:
            c = parse_model_id(model_id)
        except ValueError:
            return False
        return c.hub_name == self.hub_name or c.hub_name in self.aliases

    def _download(self, url: str, progress: Optional[Callable[[float], None]]) -> bytes:
        status, hdr, body = self._request("GET", url)
        if status != 200:
            raise HubError(f"failed to download {url}: HTTP {status}")
        if progress is not None:
            progress(100.0)
        return body

    # interface
    def get_model_metadata(self, model_id: str) -> HubModelMetadata:
        raise NotImplementedError

    def download_model(self, model_id: str, progress=None) -> bytes:
        raise NotImplementedError

    def model_exists(self, model_id: str) -> bool:
        raise NotImplementedError

    def list_models(self, filter: Optional[str] = None) -> List[str]:
        raise NotImplementedError


def _bare(model_id: str) -> str:
    """``hub:hf/org/name`` -> ``org/name``; ids without the prefix pass through."""
    if not model_id.startswith("hub:"):
        return model_id
    rest = model_id[4:]
    sep = min([i for i in (rest.find(":"), rest.find("/")) if i >= 0], default=-1)
    return rest[sep + 1:] if sep >= 0 else rest


class HuggingFaceHub(ModelHub):
    hub_name, aliases = "huggingface", ("hf",)

    def __init__(self, configuration: Optional[HuggingFaceHubConfiguration] = None, authentication=None, transport=None, sleep=time.sleep):
        cfg = configuration or HuggingFaceHubConfiguration()
        if authentication is None and cfg.api_token:
            authentication = TokenAuth(cfg.api_token)
        super().__init__(cfg, authentication, transport, sleep)

    def get_model_metadata(self, model_id: str) -> HubModelMetadata:
        repo = _bare(model_id)
        status, _, body = self._request("GET", f"{self.configuration.effective_base_url}/api/models/{repo}")
        if status != 200:
            raise HubError(f"failed to get metadata for model {repo!r}: HTTP {status}")
        info = json.loads(body.decode() or "{}")
        card = info.get("cardData") or {}
        return HubModelMetadata(info.get("modelId") or info.get("id") or repo, card.get("description") or info.get("description") or "",
                                info.get("library_name") or "pytorch", (info.get("config") or {}).get("model_type") or info.get("model_type") or "unknown",
                                {"hub": self.hub_name, "author": info.get("author") or "unknown", "downloads": str(info.get("downloads", 0)),
                                 "likes": str(info.get("likes", 0)), "lastModified": info.get("lastModified") or "",
                                 "files": ",".join(s.get("rfilename", "") for s in info.get("siblings") or [])})

    def download_model(self, model_id: str, progress=None, filename: Optional[str] = None, revision: str = "main") -> bytes:
        repo = _bare(model_id)
        if filename is None:
            files = [f for f in self.get_model_metadata(model_id).custom.get("files", "").split(",") if f]
            prefer = [f for f in files if f.endswith(".safetensors")] or [f for f in files if f.endswith(".bin")] or files
            if not prefer:
                raise HubError(f"model {repo!r} lists no files")
            filename = prefer[0]
        return self._download(f"{self.configuration.effective_base_url}/{repo}/resolve/{revision}/{filename}", progress)

    def model_exists(self, model_id: str) -> bool:
        return self._request("HEAD", f"{self.configuration.effective_base_url}/api/models/{_bare(model_id)}")[0] == 200

    def list_models(self, filter: Optional[str] = None) -> List[str]:
        url = f"{self.configuration.effective_base_url}/api/models" + (f"?search={filter}" if filter else "")
        status, _, body = self._request("GET", url)
        if status != 200:
            return []
        return [m.get("modelId") or m.get("id") for m in json.loads(body.decode() or "[]")]


class TensorFlowHub(ModelHub):
    hub_name, aliases = "tensorflow", ("tfhub", "tf")

    def __init__(self, configuration: Optional[TensorFlowHubConfiguration] = None, authentication=None, transport=None, sleep=time.sleep):
        super().__init__(configuration or TensorFlowHubConfiguration(), authentication, transport, sleep)

    def _url(self, model_id: str) -> str:
        path = _bare(model_id).strip("/")
        q = "?tfhub-format=compressed" if self.configuration.use_compression else ""
        return f"{self.configuration.base_url}/{path}{q}"

    def get_model_metadata(self, model_id: str) -> HubModelMetadata:
        status, hdr, _ = self._request("HEAD", self._url(model_id))
        if status != 200:
            raise HubError(f"failed to get metadata for model {_bare(model_id)!r}: HTTP {status}")
        return HubModelMetadata(_bare(model_id), framework="tensorflow", architecture=self.configuration.preferred_format,
                                custom={"hub": self.hub_name, "content_length": str(hdr.get("Content-Length", "")),
                                        "compression": self.configuration.compression_format if self.configuration.use_compression else "none"})

    def download_model(self, model_id: str, progress=None) -> bytes:
        return self._download(self._url(model_id), progress)

    def model_exists(self, model_id: str) -> bool:
        return self._request("HEAD", self._url(model_id))[0] == 200

    def list_models(self, filter: Optional[str] = None) -> List[str]:
        return []          # tfhub.dev has no listing endpoint (the reference returns an empty list as well)


class ONNXHub(ModelHub):
    hub_name, aliases = "onnx", ("onnxzoo",)

    def __init__(self, configuration: Optional[ONNXHubConfiguration] = None, authentication=None, transport=None, sleep=time.sleep):
        super().__init__(configuration or ONNXHubConfiguration(), authentication, transport, sleep)

    def _parts(self, model_id: str) -> Tuple[str, str]:
        c = parse_model_id(model_id) if model_id.startswith("hub:") else ModelIdComponents(model_name=model_id)
        return c.model_name, c.version or self.configuration.default_version

    def _base(self) -> str:
        c = self.configuration
        return c.mirror_urls[0] if c.prefer_mirrors and c.mirror_urls else c.raw_content_url

    def get_model_metadata(self, model_id: str) -> HubModelMetadata:
        name, ver = self._parts(model_id)
        status, _, body = self._request("GET", f"{self.configuration.raw_content_url}/validated/vision/{ver}/{name}/data/config.json")
        if status != 200:
            raise HubError(f"failed to get metadata for model {name!r}: HTTP {status}")
        info = json.loads(body.decode() or "{}")
        return HubModelMetadata(name, info.get("description", ""), "onnx", info.get("architecture", name),
                                {"hub": self.hub_name, "version": ver, "opset": str(info.get("opset", ""))})

    def download_model(self, model_id: str, progress=None) -> bytes:
        name, ver = self._parts(model_id)
        return self._download(f"{self._base()}/validated/vision/{ver}/{name}/model/{name}.onnx", progress)

    def model_exists(self, model_id: str) -> bool:
        name, ver = self._parts(model_id)
        return self._request("HEAD", f"{self.configuration.raw_content_url}/validated/vision/{ver}/{name}/model/{name}.onnx")[0] == 200

    def list_models(self, filter: Optional[str] = None) -> List[str]:
        status, _, body = self._request("GET", f"{self.configuration.raw_content_url}/validated/vision/master")
        if status != 200:
            return []
        names = [ln.strip() for ln in body.decode().splitlines() if ln.strip()]
        return [n for n in names if not filter or filter.lower() in n.lower()]


class HubRegistry:
    def __init__(self):
        self._hubs: Dict[str, ModelHub] = {}
        self._default: Optional[str] = None

    def register_hub(self, hub: ModelHub):
        if hub.hub_name in self._hubs:
            raise ValueError(f"hub {hub.hub_name!r} is already registered")
        self._hubs[hub.hub_name] = hub
        if self._default is None:
            self._default = hub.hub_name

    def unregister_hub(self, name: str) -> bool:
        if self._hubs.pop(name, None) is None:
            return False
        if self._default == name:
            self._default = next(iter(self._hubs), None)
        return True

    def get_hub(self, name: str) -> Optional[ModelHub]:
        return self._hubs.get(name)

    def get_hub_for_model(self, model_id: str) -> Optional[ModelHub]:
        for h in self._hubs.values():
            if h.can_handle(model_id):
                return h
        return None

    def list_hubs(self) -> List[str]:
        return list(self._hubs)

    def get_default_hub(self) -> Optional[ModelHub]:
        return self._hubs.get(self._default) if self._default else None

    def set_default_hub(self, name: str) -> bool:
        if name not in self._hubs:
            return False
        self._default = name
        return True

    def is_hub_registered(self, name: str) -> bool:
        return name in self._hubs

    @property
    def count(self) -> int:
        return len(self._hubs)

    def clear(self):
        self._hubs.clear()
        self._default = None

    def register_default_hubs(self, transport: Optional[Transport] = None):
        for cls in (HuggingFaceHub, TensorFlowHub, ONNXHub):
            if cls.hub_name not in self._hubs:
                self.register_hub(cls(transport=transport))

    def download(self, model_id: str, progress=None) -> bytes:
        """Routes ``hub:...`` ids to the hub that handles them."""
        hub = self.get_hub_for_model(model_id)
        if hub is None:
            raise HubError(f"no registered hub handles {model_id!r}")
        return hub.download_model(model_id, progress)
