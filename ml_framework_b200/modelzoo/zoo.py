"""Model zoo: registry of architectures and weights, local cache, loading (full or progressive),
discovery with memory / latency estimates, transfer-learning helpers, benchmarking.

Reference (src/ModelZoo/): ModelZoo.cs, ModelRegistry.cs, ModelDownloadService.cs, ModelCacheManager.cs (file
locks, LRU), LoadFlow.cs, Serialization/*, Discovery/* (search, recommendation, latency and memory
estimators), ExternalHubs/* (HuggingFace / TF-Hub / ONNX adapters), Plugins/* (registry plug-ins with auth),
Progressive/* (lazy per-layer loading), TransferLearning/* (freeze, head replacement, layer-wise LR, gradual
unfreezing), Benchmark/*.

There is no network on the target machines, so a "download" resolves ``file://`` sources and plain paths
(other schemes raise with the reason); external hubs are adapters that read a local directory in the
hub's layout (``config.json`` + weight shards).
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import time
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .errors import ChecksumMismatchError, DownloadFailedError, ModelNotFoundError, VersionNotFoundError


@dataclass
class ModelInfo:
    name: str
    architecture: str                      # gpt | llama | mlp
    config: Dict[str, Any]
    version: str = "1.0.0"
    task: str = "causal-lm"
    source: Optional[str] = None           # weights location (path or file:// URL); None = random init
    sha256: Optional[str] = None
    tags: Tuple[str, ...] = ()
    description: str = ""
    license: str = ""
    metrics: Optional[Dict[str, float]] = None       # e.g. {"accuracy": 0.76, "perplexity": 12.3}
    file_size: Optional[int] = None                  # bytes of the weight file when known
    pretrained_dataset: str = ""
    framework_version: str = ""

    def num_params(self) -> int:
        return _build_config(self).num_params() if self.architecture in ("gpt", "llama") else 0


def _build_config(info: ModelInfo):
    if info.architecture == "gpt":
        from ..models.gpt import GPTConfig
        return GPTConfig(**info.config)
    if info.architecture == "llama":
        from ..models.llama import LlamaConfig
        return LlamaConfig(**info.config)
    raise KeyError(f"unknown architecture {info.architecture!r}")


def _version_key(v: str):
    """Orders versions: numeric fields compare as numbers, a pre-release ("1.2.0-rc.1") comes before its
    release, anything unparsable sorts lowest by its text."""
    core, _, pre = v.split("+")[0].partition("-")
    nums = []
    for part in core.split(".")[:3]:
        digits = "".join(ch for ch in part if ch.isdigit())
        if not digits:
            return (0, (), 0, v)
        nums.append(int(digits))
    return (1, tuple(nums), 0 if pre else 1, pre)


class ZooRegistry:
    def __init__(self):
        self._m: Dict[Tuple[str, str], ModelInfo] = {}
        self._plugins: List["RegistryPlugin"] = []

    def register(self, info: ModelInfo):
        self._m[(info.name, info.version)] = info

    def get(self, name: str, version: Optional[str] = None) -> ModelInfo:
        if version is not None:
            if (name, version) in self._m:
                return self._m[(name, version)]
        else:
            vs = sorted((v for n, v in self._m if n == name), key=_version_key)
            if vs:
                return self._m[(name, vs[-1])]
        for p in self._plugins:
            info = p.lookup(name, version)
            if info is not None:
                return info
        known = sorted(v for n, v in self._m if n == name)
        if version is not None and known:
            raise VersionNotFoundError(name, version, known)
        raise ModelNotFoundError(name)

    def list(self) -> List[ModelInfo]:
        return list(self._m.values())

    def add_plugin(self, p: "RegistryPlugin"):
        self._plugins.append(p)

    def search(self, text: str = "", task: Optional[str] = None, tags: Sequence[str] = (), max_params: Optional[int] = None) -> List[ModelInfo]:
        out = []
        for i in self._m.values():
            if text and text.lower() not in (i.name + " " + i.description).lower():
                continue
            if task and i.task != task:
                continue
            if any(t not in i.tags for t in tags):
                continue
            if max_params is not None and i.num_params() > max_params:
                continue
            out.append(i)
        return sorted(out, key=lambda i: i.num_params())


class RegistryPlugin:
    """A further source of model descriptions (a directory of ``*.json`` cards, optionally token-protected)."""

    def __init__(self, directory: str, token: Optional[str] = None, expected_token: Optional[str] = None):
        self.dir, self.token, self.expected = directory, token, expected_token

    def lookup(self, name: str, version: Optional[str]) -> Optional[ModelInfo]:
        if self.expected is not None and self.token != self.expected:
            raise PermissionError("registry plug-in: authentication failed")
        p = os.path.join(self.dir, f"{name}.json")
        if not os.path.exists(p):
            return None
        with open(p) as f:
            d = json.load(f)
        d["tags"] = tuple(d.get("tags", ()))
        info = ModelInfo(**d)
        return info if version in (None, info.version) else None


# ------------------------------------------------------------------ cache + download
class ModelCacheManager:
    """Directory cache keyed by name/version with an index, per-entry file locks and LRU eviction by bytes."""

    def __init__(self, root: str, max_bytes: int = 200 << 30):
        self.root, self.max_bytes = root, max_bytes
        self.hits = self.loads = 0                  # fetches served from the cache / all fetches
        os.makedirs(root, exist_ok=True)
        self._index_path = os.path.join(root, "index.json")

    def _index(self) -> Dict[str, Dict[str, Any]]:
        if os.path.exists(self._index_path):
            with open(self._index_path) as f:
                return json.load(f)
        return {}

    def _save(self, idx):
        tmp = self._index_path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(idx, f, indent=1)
        os.replace(tmp, self._index_path)

    def path(self, name: str, version: str) -> str:
        return os.path.join(self.root, f"{name}-{version}.pt")

    def lock(self, name: str, version: str):
        cache = self

        class _L:
            def __enter__(self):
                self.f = open(cache.path(name, version) + ".lock", "w")
                fcntl.flock(self.f, fcntl.LOCK_EX)

            def __exit__(self, *a):
                fcntl.flock(self.f, fcntl.LOCK_UN)
                self.f.close()
        return _L()

    def contains(self, name: str, version: str) -> bool:
        return os.path.exists(self.path(name, version))

    def touch(self, name: str, version: str):
        idx = self._index()
        key = f"{name}-{version}"
        idx.setdefault(key, {})["last_used"] = time.time()
        idx[key]["bytes"] = os.path.getsize(self.path(name, version))
        idx[key]["access_count"] = idx[key].get("access_count", 0) + 1
        self._save(idx)

    def evict(self) -> List[str]:
        idx = self._index()
        total = sum(e.get("bytes", 0) for e in idx.values())
        gone = []
        for key, e in sorted(idx.items(), key=lambda kv: kv[1].get("last_used", 0)):
            if total <= self.max_bytes:
                break
            p = os.path.join(self.root, key + ".pt")
            if os.path.exists(p):
                os.remove(p)
            total -= e.get("bytes", 0)
            gone.append(key)
        for k in gone:
            idx.pop(k)
        self._save(idx)
        return gone


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for c in iter(lambda: f.read(1 << 20), b""):
            h.update(c)
    return h.hexdigest()


class ModelDownloadService:
    def __init__(self, cache: ModelCacheManager, retries: int = 3):
        self.cache, self.retries = cache, retries

    def fetch(self, info: ModelInfo, progress: Optional[Callable[[int, int], None]] = None) -> str:
        dst = self.cache.path(info.name, info.version)
        with self.cache.lock(info.name, info.version):
            self.cache.loads += 1
            if self.cache.contains(info.name, info.version):
                self.cache.hits += 1
            else:
                src = info.source or ""
                if src.startswith("file://"):
                    src = src[7:]
                elif "://" in src:
                    raise ConnectionError(f"cannot fetch {src}: no network access; place the file locally and use a path or file:// URL")
                if not os.path.exists(src):
                    raise FileNotFoundError(f"weights for {info.name} not found at {src!r}")
                last = None
                for _ in range(self.retries):
                    try:
                        total = os.path.getsize(src)
                        with open(src, "rb") as fi, open(dst + ".part", "wb") as fo:
                            done = 0
                            for c in iter(lambda: fi.read(8 << 20), b""):
                                fo.write(c)
                                done += len(c)
                                if progress:
                                    progress(done, total)
                        os.replace(dst + ".part", dst)
                        last = None
                        break
                    except OSError as e:
                        last = e
                if last is not None:
                    raise DownloadFailedError([src], self.retries, f"{info.name}: copying {src!r} failed {self.retries} times: {last}") from last
            actual = sha256_file(dst) if info.sha256 else None
            if info.sha256 and actual != info.sha256:
                os.remove(dst)
                raise ChecksumMismatchError(dst, info.sha256, actual)
            self.cache.touch(info.name, info.version)
        self.cache.evict()
        return dst


# ------------------------------------------------------------------ loading
def build_model(info: ModelInfo, device="cpu", dtype=torch.float32) -> nn.Module:
    cfg = _build_config(info)
    if info.architecture == "gpt":
        from ..models.gpt import GPT
        return GPT(cfg).to(device=device, dtype=dtype)
    from ..models.llama import Llama
    return Llama(cfg).to(device=device, dtype=dtype)


class ProgressiveLoader:
    """Loads a state dict into a model one top-level block at a time (peak host memory = one block), calling
    ``on_layer(name, index, total)`` after each."""

    def __init__(self, state_path: str):
        self.path = state_path

    def load_into(self, model: nn.Module, on_layer: Optional[Callable[[str, int, int], None]] = None, strict: bool = True) -> List[str]:
        sd = torch.load(self.path, map_location="cpu", mmap=True, weights_only=True)
        own = dict(model.state_dict())
        groups: Dict[str, List[str]] = {}
        for k in sd:
            groups.setdefault(".".join(k.split(".")[:2]) if k.split(".")[0] in ("blocks", "layers") else k.split(".")[0], []).append(k)
        missing = [k for k in own if k not in sd]
        if strict and missing:
            raise KeyError(f"missing keys: {missing[:5]}...")
        names = list(groups)
        with torch.no_grad():
            for i, g in enumerate(names):
                for k in groups[g]:
                    if k in own:
                        own[k].copy_(sd[k])
                if on_layer:
                    on_layer(g, i, len(names))
        return missing


class ModelZoo:
    def __init__(self, cache_dir: str = "~/.cache/mlf_zoo", registry: Optional[ZooRegistry] = None):
        self.registry = registry or default_registry()
        self.cache = ModelCacheManager(os.path.expanduser(cache_dir))
        self.downloads = ModelDownloadService(self.cache)

    def load(self, name: str, version: Optional[str] = None, device="cpu", dtype=torch.float32, pretrained: bool = True,
             progressive: bool = False) -> nn.Module:
        info = self.registry.get(name, version)
        model = build_model(info, device, dtype)
        if pretrained and info.source:
            path = self.downloads.fetch(info)
            if progressive:
                ProgressiveLoader(path).load_into(model)
            else:
                model.load_state_dict(torch.load(path, map_location="cpu", weights_only=True))
        return model

    def load_progressive(self, name: str, version: Optional[str] = None, options=None, device="cpu",
                         dtype: Optional[torch.dtype] = None):
        """The model on ``meta`` with a ``progressive.ProgressiveModelLoader`` attached: layers come in
        from the cached weight file as the forward pass (or the chosen background strategy) wants
        them. Returns (model, loader)."""
        from .progressive import load_progressive
        info = self.registry.get(name, version)
        if not info.source:
            raise ValueError(f"model {name!r} has no weights to load progressively")
        path = self.downloads.fetch(info)
        return load_progressive(lambda: build_model(info, "meta", dtype or torch.float32), path, options, device, dtype, info)

    def save(self, model: nn.Module, info: ModelInfo, path: str) -> ModelInfo:
        torch.save(model.state_dict(), path)
        info.source, info.sha256 = path, sha256_file(path)
        self.registry.register(info)
        return info

    # ---- discovery
    @staticmethod
    def estimate_memory_bytes(info: ModelInfo, dtype_bytes: int = 2, training: bool = False, batch_tokens: int = 0) -> int:
        p = info.num_params()
        weights = p * dtype_bytes
        if not training:
            return weights
        d = info.config.get("d_model", 0)
        L = info.config.get("n_layers", 0)
        return weights + p * dtype_bytes + p * 12 + batch_tokens * d * L * 34    # grads + fp32 master/m/v + activations

    @staticmethod
    def estimate_latency_ms(info: ModelInfo, tokens: int = 1, tflops: float = 1400.0, hbm_gbs: float = 6500.0, dtype_bytes: int = 2) -> float:
        p = info.num_params()
        return max(2.0 * p * tokens / (tflops * 1e12), p * dtype_bytes / (hbm_gbs * 1e9)) * 1e3

    def recommend(self, memory_budget_bytes: int, task: str = "causal-lm") -> Optional[ModelInfo]:
        fits = [i for i in self.registry.search(task=task) if self.estimate_memory_bytes(i) <= memory_budget_bytes]
        return fits[-1] if fits else None

    def benchmark(self, name: str, batch: int = 1, seq: int = 128, device="cpu", iters: int = 3) -> Dict[str, float]:
        info = self.registry.get(name)
        dt = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
        m = build_model(info, device, dt).eval()
        ids = torch.randint(0, info.config.get("vocab_size", 100), (batch, seq), device=device)
        with torch.no_grad():
            m(ids)
            t0 = time.perf_counter()
            for _ in range(iters):
                m(ids)
            if str(device).startswith("cuda"):
                torch.cuda.synchronize()
        dt_s = (time.perf_counter() - t0) / iters
        return {"ms": dt_s * 1e3, "tokens_per_s": batch * seq / dt_s}


class LocalHubAdapter:
    """Reads a directory in the HuggingFace layout (``config.json`` with ``hidden_size`` etc.) into a ``ModelInfo``."""
    KEYS = {"llama": {"n_layers": "num_hidden_layers", "d_model": "hidden_size", "n_heads": "num_attention_heads", "n_kv_heads": "num_key_value_heads",
                      "d_ff": "intermediate_size", "vocab_size": "vocab_size", "max_seq": "max_position_embeddings", "rope_theta": "rope_theta",
                      "norm_eps": "rms_norm_eps"},
            "gpt": {"n_layers": "n_layer", "d_model": "n_embd", "n_heads": "n_head", "vocab_size": "vocab_size", "max_seq": "n_positions"}}

    def info_from_dir(self, directory: str, name: Optional[str] = None) -> ModelInfo:
        with open(os.path.join(directory, "config.json")) as f:
            c = json.load(f)
        arch = "llama" if "llama" in str(c.get("model_type", "")).lower() else "gpt"
        cfg = {k: c[v] for k, v in self.KEYS[arch].items() if v in c}
        if arch == "llama":
            cfg["head_dim"] = c.get("head_dim", cfg["d_model"] // cfg["n_heads"])
        else:
            cfg["d_ff"] = c.get("n_inner") or 4 * cfg["d_model"]
        return ModelInfo(name or os.path.basename(directory.rstrip("/")), arch, cfg, source=None, tags=("hub",))


# ------------------------------------------------------------------ transfer learning
def freeze(model: nn.Module, patterns: Sequence[str] = ("",)) -> int:
    n = 0
    for name, p in model.named_parameters():
        if any(pt in name for pt in patterns):
            p.requires_grad_(False)
            n += 1
    return n


def unfreeze(model: nn.Module, patterns: Sequence[str] = ("",)) -> int:
    n = 0
    for name, p in model.named_parameters():
        if any(pt in name for pt in patterns):
            p.requires_grad_(True)
            n += 1
    return n


def replace_head(model: nn.Module, attr: str, new_head: nn.Module) -> nn.Module:
    if not hasattr(model, attr):
        raise AttributeError(f"model has no attribute {attr!r}")
    setattr(model, attr, new_head)
    return model


def layerwise_lr_groups(model: nn.Module, base_lr: float, decay: float = 0.9, blocks_attr: str = "blocks") -> List[Dict[str, Any]]:
    """Parameter groups with lr = base_lr * decay^(depth from the top): the last block trains fastest."""
    blocks = list(getattr(model, blocks_attr))
    L = len(blocks)
    groups, seen = [], set()
    for i, b in enumerate(blocks):
        ps = [p for p in b.parameters() if p.requires_grad]
        seen.update(id(p) for p in ps)
        groups.append({"params": ps, "lr": base_lr * decay ** (L - 1 - i), "name": f"{blocks_attr}.{i}"})
    rest = [p for p in model.parameters() if p.requires_grad and id(p) not in seen]
    groups.append({"params": rest, "lr": base_lr, "name": "rest"})
    return groups


class GradualUnfreezer:
    """Starts with only the head trainable; ``step_epoch`` unfreezes ``per_epoch`` more blocks from the top."""

    def __init__(self, model: nn.Module, blocks_attr: str = "blocks", per_epoch: int = 1):
        self.blocks, self.k, self.unfrozen = list(getattr(model, blocks_attr)), per_epoch, 0
        for b in self.blocks:
            for p in b.parameters():
                p.requires_grad_(False)

    def step_epoch(self) -> int:
        for b in self.blocks[len(self.blocks) - self.unfrozen - self.k:len(self.blocks) - self.unfrozen]:
            for p in b.parameters():
                p.requires_grad_(True)
        self.unfrozen = min(len(self.blocks), self.unfrozen + self.k)
        return self.unfrozen


def default_registry() -> ZooRegistry:
    r = ZooRegistry()
    r.register(ModelInfo("gpt-125m", "gpt", dict(n_layers=12, d_model=768, n_heads=6, d_ff=3072, vocab_size=50257, max_seq=2048),
                         tags=("gpt", "small"), description="GPT-style decoder, 125 M parameters, head dim 128"))
    r.register(ModelInfo("gpt-1.3b", "gpt", dict(n_layers=24, d_model=2048, n_heads=16, d_ff=8192, vocab_size=50257, max_seq=2048),
                         tags=("gpt", "benchmark"), description="GPT-style decoder, 1.3 B parameters (training benchmark)"))
    r.register(ModelInfo("llama-3-8b", "llama", dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=14336,
                                                     vocab_size=128256, max_seq=8192), tags=("llama", "serving"),
                         description="Llama-3-8B architecture (serving benchmark)"))
    r.register(ModelInfo("llama-2-13b", "llama", dict(n_layers=40, d_model=5120, n_heads=40, n_kv_heads=40, head_dim=128, d_ff=13824,
                                                      vocab_size=32000, max_seq=4096, rope_theta=10000.0), tags=("llama",),
                         description="Llama-2-13B architecture (tensor + pipeline parallel configuration)"))
    r.register(ModelInfo("llama-tiny", "llama", dict(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, head_dim=128, d_ff=512, vocab_size=1024,
                                                     max_seq=512), tags=("llama", "test"), description="two-layer test model"))
    return r
