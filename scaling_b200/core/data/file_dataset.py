"""Same three-file format as ``MemoryMapDataset``, read with seek + read instead of mmap.

A failing network filesystem kills a process that touches an mmap'ed page (SIGBUS), whereas a
failed ``read`` raises and can be retried; this class trades some speed for that robustness
(src/scaling/core/data/file_dataset.py:11-196).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import IO, Any, Iterator, Optional

import numpy as np

from .file_handles import FileHandle, RetryableException


def retry_array_from_file(file_handle: FileHandle, dtype: np.dtype, count: int, offset: int, max_attempts: int = 5,
                          max_delay: int = 32) -> np.ndarray:
    """Read ``count`` items of ``dtype`` at byte ``offset``; short reads are treated as retryable."""
    dtype = np.dtype(dtype)

    def read(f: IO[Any]) -> np.ndarray:
        f.seek(offset)
        arr = np.fromfile(f, dtype=dtype, count=count)
        if len(arr) == 0 and count != 0:
            raise RetryableException(
                f"Expected to read {count} elements of dtype {dtype} at offset {offset} from {file_handle._path}, "
                f"but got {len(arr)}"
            )
        if len(arr) != count:
            raise RuntimeError(f"read {len(arr)} of {count} elements at offset {offset} from {file_handle._path}")
        return arr

    return file_handle.retry_operation(read, max_attempts=max_attempts, max_delay=max_delay)


class FileDataset:
    def __init__(self, prefix_path: Path, load_index_to_memory: bool = False) -> None:
        self.prefix_path = Path(prefix_path)
        self.load_index_to_memory = load_index_to_memory
        self.initialize()

    @property
    def file_path_data(self) -> Path:
        return Path(str(self.prefix_path) + ".bin")

    @property
    def file_path_index(self) -> Path:
        return Path(str(self.prefix_path) + ".idx")

    @property
    def file_path_meta(self) -> Path:
        return Path(str(self.prefix_path) + ".meta.json")

    def initialize(self) -> None:
        meta_file = FileHandle(self.file_path_meta, "r")
        meta = meta_file.retry_operation(json.load)
        meta_file.close()
        self.dtype = np.dtype(meta["dtype"])
        self.index_dtype = np.dtype(meta["index_dtype"])
        self.dtype_size = self.dtype.itemsize
        self.index_dtype_size = self.index_dtype.itemsize
        self.document_count = int(meta["document_count"])
        self._bin_file = FileHandle(self.file_path_data, "rb")
        self._index_file = FileHandle(self.file_path_index, "rb")
        self._index: Optional[np.ndarray] = None
        if self.load_index_to_memory:
            flat = retry_array_from_file(self._index_file, self.index_dtype, 2 * len(self), 0)
            self._index = np.array(flat).reshape(len(self), 2)
            self._index_file.close()

    def _entry(self, idx: int) -> tuple[int, int]:
        if self._index is not None:
            start, size = self._index[idx].tolist()
        else:
            start, size = retry_array_from_file(self._index_file, self.index_dtype, 2,
                                                int(idx) * 2 * self.index_dtype_size).tolist()
        return int(start), int(size)

    def sizes(self, idx: Optional[int] = None) -> np.ndarray:
        if idx is not None:
            return np.array(self._entry(idx)[1], dtype=self.index_dtype)
        if self._index is not None:
            return self._index[:, 1]
        return np.array([self._entry(i)[1] for i in range(len(self))], dtype=self.index_dtype)

    def __len__(self) -> int:
        return self.document_count

    def __getitem__(self, idx: int) -> np.ndarray:
        if not isinstance(idx, (int, np.integer)):
            raise NotImplementedError
        assert idx < self.document_count, f"cannot retrieve document idx {idx} from {self.document_count} documents"
        start, size = self._entry(int(idx))
        return retry_array_from_file(self._bin_file, self.dtype, size, start * self.dtype_size)

    def __iter__(self) -> Iterator[np.ndarray]:
        for i in range(len(self)):
            yield self[i]

    def __del__(self) -> None:
        for name in ("_bin_file", "_index_file"):
            h = getattr(self, name, None)
            if h is not None:
                h.close()
