"""Configuration, bookkeeping and validation types of the model zoo.

Reference: src/ModelZoo/{TaskType.cs, ModelZooConfiguration.cs, CacheConfiguration.cs,
CacheMetadata.cs:10-101, CacheStatistics.cs:10-154, DownloadProgress.cs:8-98,
ModelMetadataValidator.cs:12-181, RegistryBuilder.cs:12-173}.
"""
from __future__ import annotations

import enum
import glob
import json
import os
import re
import time
from dataclasses import asdict, dataclass, field
from typing import Dict, Iterable, List, Optional

from .zoo import ModelInfo, ZooRegistry

__all__ = [
    "TaskType", "ModelZooConfiguration", "CacheConfiguration", "CacheMetadata", "ModelAccessInfo",
    "CacheStatistics", "DownloadProgress", "format_bytes", "ModelMetadataValidator", "RegistryBuilder",
    "cache_statistics",
]


class TaskType(enum.Enum):
    IMAGE_CLASSIFICATION = "image-classification"
    OBJECT_DETECTION = "object-detection"
    SEMANTIC_SEGMENTATION = "semantic-segmentation"
    TEXT_CLASSIFICATION = "text-classification"
    SEQUENCE_LABELING = "sequence-labeling"
    QUESTION_ANSWERING = "question-answering"
    TEXT_GENERATION = "causal-lm"
    REGRESSION = "regression"


@dataclass
class ModelZooConfiguration:
    default_device: str = "cpu"
    cache_enabled: bool = True
    auto_download_enabled: bool = True
    default_download_timeout_ms: int = 300_000


@dataclass
class CacheConfiguration:
    cache_root_path: str = "~/.cache/mlf_zoo"
    max_cache_size_bytes: int = 10 << 30
    max_file_age_s: float = 30 * 86400.0
    cleanup_on_startup: bool = False
    lock_timeout_ms: int = 30_000


def format_bytes(n: float) -> str:
    units = ["B", "KB", "MB", "GB", "TB"]
    i, size = 0, float(n)
    while size >= 1024 and i < len(units) - 1:
        size /= 1024
        i += 1
    text = f"{size:.2f}".rstrip("0").rstrip(".")
    return f"{text} {units[i]}"


@dataclass
class CacheMetadata:
    """What the cache remembers about one file."""
    model_name: str = ""
    version: str = ""
    file_size: int = 0
    access_count: int = 0
    checksum: Optional[str] = None
    last_accessed: float = field(default_factory=time.time)
    download_date: float = field(default_factory=time.time)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @classmethod
    def from_json(cls, text: str) -> "CacheMetadata":
        d = json.loads(text)
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in known})

    def record_access(self, now: Optional[float] = None) -> None:
        self.last_accessed = time.time() if now is None else now
        self.access_count += 1


@dataclass
class ModelAccessInfo:
    model_name: str = ""
    version: str = ""
    last_accessed: float = 0.0
    access_count: int = 0
    file_size: int = 0


@dataclass
class CacheStatistics:
    total_models: int = 0
    total_cache_size: int = 0
    cache_hits: int = 0
    total_loads: int = 0
    least_recently_used: List[ModelAccessInfo] = field(default_factory=list)
    most_recently_used: List[ModelAccessInfo] = field(default_factory=list)

    @property
    def cache_hit_rate(self) -> float:
        return self.cache_hits / self.total_loads if self.total_loads else 0.0

    def record_hit(self) -> None:
        self.cache_hits += 1
        self.total_loads += 1

    def record_miss(self) -> None:
        self.total_loads += 1

    def summary(self) -> str:
        return (f"cache: {self.total_models} models, {format_bytes(self.total_cache_size)}, "
                f"{self.cache_hits} hits of {self.total_loads} loads ({self.cache_hit_rate * 100:.2f} %)")


def cache_statistics(cache, top: int = 5) -> CacheStatistics:
    """Statistics of a ``zoo.ModelCacheManager`` from its index (hits and loads as it counted them)."""
    idx = cache._index()
    infos = []
    for key, e in idx.items():
        name, _, version = key.rpartition("-")
        infos.append(ModelAccessInfo(name, version, e.get("last_used", 0.0), e.get("access_count", 0), e.get("bytes", 0)))
    infos.sort(key=lambda i: i.last_accessed)
    return CacheStatistics(len(infos), sum(i.file_size for i in infos), getattr(cache, "hits", 0), getattr(cache, "loads", 0),
                           infos[:top], infos[::-1][:top])


@dataclass
class DownloadProgress:
    bytes_downloaded: int = 0
    total_bytes: int = 0
    current_url: str = ""
    download_speed: float = 0.0                   # bytes per second

    @property
    def progress_percentage(self) -> float:
        return self.bytes_downloaded / self.total_bytes if self.total_bytes > 0 else 0.0

    @property
    def estimated_time_remaining_s(self) -> Optional[float]:
        if self.download_speed <= 0 or self.total_bytes <= 0:
            return None
        return max(0, self.total_bytes - self.bytes_downloaded) / self.download_speed

    @property
    def progress_percentage_text(self) -> str:
        return f"{self.progress_percentage * 100:.1f}%"

    @property
    def bytes_downloaded_text(self) -> str:
        return format_bytes(self.bytes_downloaded)

    @property
    def total_bytes_text(self) -> str:
        return format_bytes(self.total_bytes)

    @property
    def download_speed_text(self) -> str:
        return f"{format_bytes(self.download_speed)}/s"

    @classmethod
    def tracker(cls, url: str, callback, clock=time.monotonic):
        """A ``progress(done, total)`` function for ``ModelDownloadService.fetch`` that turns byte
        counts into ``DownloadProgress`` records (speed averaged since the first call)."""
        t0 = [None]

        def progress(done: int, total: int):
            now = clock()
            if t0[0] is None:
                t0[0] = (now, done)
            dt = now - t0[0][0]
            speed = (done - t0[0][1]) / dt if dt > 0 else 0.0
            callback(cls(done, total, url, speed))
        return progress


_SEMVER = re.compile(r"^\d+\.\d+\.\d+(?:-[0-9A-Za-z.-]+)?(?:\+[0-9A-Za-z.-]+)?$")
_URL = re.compile(r"^(?:https?|file|s3|gs)://\S+$")
_SHA256 = re.compile(r"^[0-9a-fA-F]{64}$")
_UNIT_METRICS = {"accuracy", "precision", "recall", "f1", "f1_score", "auc", "map", "iou", "miou", "bleu_normalized"}
_ARCHITECTURES = ("gpt", "llama", "mlp", "local", "remote")


class ModelMetadataValidator:
    """Checks a model card before it enters a registry (ModelMetadataValidator.cs:36-181)."""

    @staticmethod
    def validate(info: Optional[ModelInfo]) -> List[str]:
        if info is None:
            return ["metadata cannot be None"]
        errors: List[str] = []
        if not info.name or not info.name.strip():
            errors.append("name is required")
        if not info.architecture:
            errors.append("architecture is required")
        if not info.version or not _SEMVER.match(info.version):
            errors.append(f"version '{info.version}' does not follow semantic versioning")
        src = info.source
        if src and "://" in src and not _URL.match(src):
            errors.append(f"source '{src}' is not a valid URL")
        if info.sha256 and not _SHA256.match(info.sha256):
            errors.append(f"sha256 '{info.sha256}' is not a 64-character hex string")
        for k, v in (info.metrics or {}).items():
            name = k.lower()
            if not isinstance(v, (int, float)) or v != v:
                errors.append(f"metric '{k}' is not a number")
                continue
            if (name in _UNIT_METRICS or name.startswith("top")) and not 0 <= v <= 1:
                errors.append(f"metric '{k}' has value {v} but should lie in [0, 1]")
            elif v < 0:
                errors.append(f"metric '{k}' has negative value {v}")
        if info.file_size is not None and info.file_size < 0:
            errors.append("file size cannot be negative")
        if info.architecture in ("gpt", "llama"):
            if not isinstance(info.config, dict) or not info.config:
                errors.append(f"a {info.architecture} card needs a config")
            else:
                for k, v in info.config.items():
                    if isinstance(v, int) and not isinstance(v, bool) and v < 0:
                        errors.append(f"config field '{k}' cannot be negative")
        return errors

    @classmethod
    def validate_or_raise(cls, info: ModelInfo) -> None:
        errors = cls.validate(info)
        if errors:
            raise ValueError("invalid model metadata: " + "; ".join(errors))

    @classmethod
    def is_valid(cls, info: ModelInfo) -> bool:
        return not cls.validate(info)


def _info_from_dict(d: Dict) -> ModelInfo:
    d = dict(d)
    d["tags"] = tuple(d.get("tags", ()))
    known = set(ModelInfo.__dataclass_fields__)
    unknown = set(d) - known
    if unknown:
        raise KeyError(f"unknown card fields: {sorted(unknown)}")
    return ModelInfo(**d)


class RegistryBuilder:
    """Collects cards from objects, JSON files and directories; ``build`` validates them and refuses
    the same (name, version) twice (RegistryBuilder.cs:12-173)."""

    def __init__(self):
        self._cards: List[ModelInfo] = []

    @property
    def count(self) -> int:
        return len(self._cards)

    def add(self, info: ModelInfo) -> "RegistryBuilder":
        if info is None:
            raise ValueError("the card is required")
        self._cards.append(info)
        return self

    def add_range(self, infos: Iterable[ModelInfo]) -> "RegistryBuilder":
        for i in infos:
            self.add(i)
        return self

    def add_from_json_file(self, path: str) -> "RegistryBuilder":
        """A file holding one card or a list of cards."""
        if not os.path.isfile(path):
            raise FileNotFoundError(path)
        try:
            with open(path) as f:
                data = json.load(f)
            for d in (data if isinstance(data, list) else [data]):
                self.add(_info_from_dict(d))
        except (ValueError, KeyError, TypeError) as e:
            raise ValueError(f"cannot load model metadata from {path}: {e}") from e
        return self

    def add_from_directory(self, path: str) -> "RegistryBuilder":
        if not os.path.isdir(path):
            raise FileNotFoundError(f"directory not found: {path}")
        for p in sorted(glob.glob(os.path.join(path, "*.json"))):
            self.add_from_json_file(p)
        return self

    def build(self, validate: bool = True) -> ZooRegistry:
        reg = ZooRegistry()
        seen = set()
        for c in self._cards:
            if validate:
                errors = ModelMetadataValidator.validate(c)
                if errors:
                    raise ValueError(f"cannot register model '{c.name}' version '{c.version}': " + "; ".join(errors))
            if (c.name, c.version) in seen:
                raise ValueError(f"model '{c.name}' version '{c.version}' appears twice")
            seen.add((c.name, c.version))
            reg.register(c)
        return reg

    def clear(self) -> None:
        self._cards.clear()
