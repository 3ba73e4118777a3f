"""File handle whose operations are retried on stale-NFS errors.

``retry_operation`` re-opens the file and repeats the operation when it fails with ``ESTALE`` or a
``RetryableException``, with exponential back-off (at most ``max_attempts`` tries, delays capped at
``max_delay`` seconds); any other error propagates at once
(behaviour of src/scaling/core/data/file_handles.py:9-70).  ``sleep`` can be replaced in tests.
"""

from __future__ import annotations

import time
from errno import ESTALE
from pathlib import Path
from typing import IO, Any, Callable, Optional, TypeVar

V = TypeVar("V")


class RetryableException(Exception):
    pass


def is_retryable(e: BaseException) -> bool:
    if isinstance(e, OSError):
        return e.errno == ESTALE
    return isinstance(e, RetryableException)


class FileHandle:
    sleep: Callable[[float], None] = staticmethod(time.sleep)

    def __init__(self, path: Path, mode: str = "rb"):
        self._path = Path(path)
        self._mode = mode
        self._handle: Optional[IO[Any]] = None

    def _open(self) -> IO[Any]:
        if self._handle is None:
            self._handle = open(self._path, self._mode)
        return self._handle

    def retry_operation(self, func: Callable[[IO[Any]], V], max_attempts: int = 5, max_delay: int = 32) -> V:
        for attempt in range(1, max_attempts + 1):
            try:
                return func(self._open())
            except Exception as e:
                if not is_retryable(e):
                    raise
                try:
                    self.close()
                except Exception as close_error:
                    print(f"closing {self._path} failed: {close_error}", flush=True)
                print(f"retryable error on {self._path}: {e} (attempt {attempt}/{max_attempts})", flush=True)
                if attempt < max_attempts:
                    self.sleep(min(2 ** attempt, max_delay))
        raise Exception(f"Stale file handle even after {max_attempts} retries for {self._path}.")

    def close(self) -> None:
        if self._handle is not None:
            self._handle.close()
            self._handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
