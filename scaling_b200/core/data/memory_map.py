"""Token storage as three files: ``{prefix}.bin`` (all documents back to back), ``{prefix}.idx``
(pairs ``[start, length]`` per document) and ``{prefix}.meta.json`` (``dtype``, ``index_dtype``,
``document_count``) - the on-disk format of src/scaling/core/data/memory_map.py:8-250.

Reads go through ``numpy.memmap`` views, so opening a multi-terabyte dataset costs nothing and a
document access touches only its own pages; the index can optionally be pulled into memory.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterator, Optional

import numpy as np


class MemoryMapDataset:
    def __init__(self, prefix_path: Path, load_index_to_memory: bool = False) -> None:
        self.prefix_path = Path(prefix_path)
        self.load_index_to_memory = load_index_to_memory
        for f in (self.file_path_data, self.file_path_index, self.file_path_meta):
            assert f.is_file(), f"cannot initialize memory map, file not found: {f}"
        self.initialize()

    # ---- file names
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
        meta = json.loads(self.file_path_meta.read_text())
        self.dtype = np.dtype(meta["dtype"])
        self.index_dtype = np.dtype(meta["index_dtype"])
        self.dtype_size = self.dtype.itemsize
        self.index_dtype_size = self.index_dtype.itemsize
        self.document_count = int(meta["document_count"])
        self._data = np.memmap(self.file_path_data, mode="r", order="C", dtype=self.dtype) \
            if self.file_path_data.stat().st_size > 0 else np.zeros(0, dtype=self.dtype)
        index = np.memmap(self.file_path_index, mode="r", order="C", dtype=self.index_dtype) \
            if self.file_path_index.stat().st_size > 0 else np.zeros(0, dtype=self.index_dtype)
        index = index[: 2 * self.document_count].reshape(self.document_count, 2)
        self._index = np.array(index) if self.load_index_to_memory else index

    def close(self) -> None:
        for name in ("_data", "_index"):
            arr = getattr(self, name, None)
            mm = getattr(arr, "_mmap", None) if arr is not None else None
            if mm is not None:
                try:
                    mm.close()
                except Exception:
                    pass
            if hasattr(self, name):
                delattr(self, name)

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    def sizes(self, idx: Optional[int] = None) -> np.ndarray:
        """Token counts of all documents, or of document ``idx``."""
        if idx is None:
            return np.array(self._index[:, 1])
        return np.array(self._index[idx, 1], dtype=self.index_dtype)

    def __len__(self) -> int:
        return self.document_count

    def __getitem__(self, idx: int) -> np.ndarray:
        if not isinstance(idx, (int, np.integer)):
            raise NotImplementedError
        assert idx < self.document_count, f"cannot retrieve document idx {idx} from {self.document_count} documents"
        start, size = (int(v) for v in self._index[idx])
        return self._data[start:start + size]

    def __iter__(self) -> Iterator[np.ndarray]:
        for i in range(len(self)):
            yield self[i]


class MemoryMapDatasetBuilder(MemoryMapDataset):
    """Appends one-dimensional arrays; ``finalize`` writes the meta file."""

    def __init__(self, prefix_path: Path, dtype: np.dtype = np.dtype(np.int32),
                 index_dtype: np.dtype = np.dtype(np.int64)):
        self.prefix_path = Path(prefix_path)
        self.dtype = np.dtype(dtype)
        self.index_dtype = np.dtype(index_dtype)
        self.initialize()

    def initialize(self) -> None:
        assert not self.file_path_data.is_file(), f"data file already exists: {self.file_path_data}"
        assert not self.file_path_index.is_file(), f"index file already exists: {self.file_path_index}"
        self.file_path_data.parent.mkdir(exist_ok=True, parents=True)
        self.data_file = open(self.file_path_data, "wb")
        self.index_file = open(self.file_path_index, "wb")
        self.current_index = 0
        self.document_count = 0

    def add(self, np_array: np.ndarray) -> None:
        assert np_array.ndim == 1, "cannot add arrays of more than one dimension"
        self.data_file.write(np.ascontiguousarray(np_array, dtype=self.dtype).tobytes(order="C"))
        self.index_file.write(np.array([self.current_index, len(np_array)], dtype=self.index_dtype).tobytes(order="C"))
        self.current_index += len(np_array)
        self.document_count += 1

    def finalize(self) -> None:
        assert not self.data_file.closed and not self.index_file.closed, "The Builder has been finalized already"
        self.data_file.close()
        self.index_file.close()
        with open(self.file_path_meta, "w") as f:
            json.dump({"dtype": self.dtype.name, "index_dtype": self.index_dtype.name,
                       "document_count": self.document_count}, f)

    def __del__(self) -> None:
        for name in ("data_file", "index_file"):
            f = getattr(self, name, None)
            if f is not None and not f.closed:
                f.close()

    def __enter__(self) -> "MemoryMapDatasetBuilder":
        return self

    def __exit__(self, *exc) -> bool:
        if not self.data_file.closed:
            self.finalize()
        return False
