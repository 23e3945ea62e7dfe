"""Errors of the model zoo, each carrying the facts a caller needs to react
(reference: src/ModelZoo/Exceptions/*.cs)."""
from __future__ import annotations

from typing import Optional, Sequence


class ModelZooError(RuntimeError):
    """Base of every error below."""


class ModelNotFoundError(ModelZooError, KeyError):
    def __init__(self, model_name: str):
        super().__init__(f"model '{model_name}' was not found in any registry")
        self.model_name = model_name

    def __str__(self):                       # KeyError would quote the message
        return self.args[0]


class VersionNotFoundError(ModelZooError, KeyError):
    def __init__(self, model_name: str, version: str, available: Sequence[str] = ()):
        tail = f" (available: {', '.join(available)})" if available else ""
        super().__init__(f"version '{version}' of model '{model_name}' was not found{tail}")
        self.model_name, self.version, self.available = model_name, version, list(available)

    def __str__(self):
        return self.args[0]


class ChecksumMismatchError(ModelZooError, IOError):
    def __init__(self, file_path: str, expected_checksum: str, actual_checksum: str):
        super().__init__(f"checksum mismatch for '{file_path}': expected {expected_checksum}, got {actual_checksum}")
        self.file_path, self.expected_checksum, self.actual_checksum = file_path, expected_checksum, actual_checksum


class DeserializationError(ModelZooError):
    def __init__(self, file_path: str, message: str):
        super().__init__(f"cannot read '{file_path}': {message}")
        self.file_path = file_path


class DownloadFailedError(ModelZooError, IOError):
    def __init__(self, attempted_urls: Sequence[str], retry_count: int, message: Optional[str] = None):
        super().__init__(message or f"download failed after {retry_count} retries from: {', '.join(attempted_urls)}")
        self.attempted_urls, self.retry_count = list(attempted_urls), retry_count


class DownloadTimeoutError(ModelZooError, TimeoutError):
    def __init__(self, url: str, timeout_ms: int, bytes_downloaded: int = 0):
        super().__init__(f"download of '{url}' timed out after {timeout_ms} ms ({bytes_downloaded} bytes received)")
        self.url, self.timeout_ms, self.bytes_downloaded = url, timeout_ms, bytes_downloaded


class IncompatibleModelError(ModelZooError):
    def __init__(self, model_name: str, version: str, expected_architecture: str, actual_architecture: str):
        super().__init__(f"model '{model_name}' version '{version}' has architecture '{actual_architecture}', "
                         f"expected '{expected_architecture}'")
        self.model_name, self.version = model_name, version
        self.expected_architecture, self.actual_architecture = expected_architecture, actual_architecture
