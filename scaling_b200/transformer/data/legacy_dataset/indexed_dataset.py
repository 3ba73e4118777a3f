"""Readers and writers for Megatron / fairseq style indexed datasets (legacy corpora)
(src/scaling/transformer/data/legacy_dataset/indexed_dataset.py:19-476).

Two on-disk layouts, each a pair ``{prefix}.bin`` (raw items back to back) + ``{prefix}.idx``:

* "mmap" (magic ``MMIDIDX\\0\\0``): version u64, dtype code u8, item count u64, document count u64, then
  ``sizes int32[n]``, ``pointers int64[n]`` (byte offsets into the .bin file), ``doc_idx int64[docs]``.
* "cached" / "lazy" (magic ``TNTIDX\\0\\0``): version u64, dtype code u64, element size u64, item count u64, size
  count u64, then ``dim_offsets int64[n + 1]``, ``data_offsets int64[n + 1]`` (in elements), ``sizes int64[s]``.
"""

from __future__ import annotations

import os
import struct
from typing import Any, Optional, Union

import numpy as np
import torch

DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
MMAP_MAGIC = b"MMIDIDX\x00\x00"
TNT_MAGIC = b"TNTIDX\x00\x00"


def dtype_code(dtype: Any) -> int:
    for code, dt in DTYPES.items():
        if np.dtype(dt) == np.dtype(dtype):
            return code
    raise ValueError(f"unsupported dtype {dtype}")


def best_fitting_dtype(vocab_size: Optional[int] = None) -> type:
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


def index_file_path(prefix_path: str) -> str:
    return prefix_path + ".idx"


def data_file_path(prefix_path: str) -> str:
    return prefix_path + ".bin"


def infer_dataset_impl(path: str) -> Optional[str]:
    """"mmap", "cached" or None, from the magic bytes of the index file."""
    if not os.path.exists(index_file_path(path)):
        return None
    with open(index_file_path(path), "rb") as f:
        magic = f.read(9)
    if magic[:8] == TNT_MAGIC:
        return "cached"
    if magic == MMAP_MAGIC:
        return "mmap"
    return None


class MMapIndexedDataset(torch.utils.data.Dataset):
    """Zero-copy reader of the "mmap" layout."""

    def __init__(self, path: str, skip_warmup: bool = True) -> None:
        self._path = path
        with open(index_file_path(path), "rb") as f:
            assert f.read(9) == MMAP_MAGIC, "index file does not match the expected mmap format"
            (version,) = struct.unpack("<Q", f.read(8))
            assert version == 1
            (code,) = struct.unpack("<B", f.read(1))
            self._dtype = np.dtype(DTYPES[code])
            (self._len,) = struct.unpack("<Q", f.read(8))
            (self._doc_count,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self._index = np.memmap(index_file_path(path), mode="r", order="C")
        self._sizes = np.frombuffer(self._index, dtype=np.int32, count=self._len, offset=offset)
        self._pointers = np.frombuffer(self._index, dtype=np.int64, count=self._len, offset=offset + self._sizes.nbytes)
        self._doc_idx = np.frombuffer(self._index, dtype=np.int64, count=self._doc_count,
                                      offset=offset + self._sizes.nbytes + self._pointers.nbytes)
        self._data = np.memmap(data_file_path(path), mode="r", order="C")

    def __len__(self) -> int:
        return int(self._len)

    @property
    def sizes(self) -> np.ndarray:
        return self._sizes

    @property
    def doc_idx(self) -> np.ndarray:
        return self._doc_idx

    @property
    def dtype(self) -> np.dtype:
        return self._dtype

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        """``length`` elements of item ``idx`` starting at element ``offset``."""
        size = int(self._sizes[idx])
        length = size - offset if length is None else length
        ptr = int(self._pointers[idx]) + offset * self._dtype.itemsize
        return np.frombuffer(self._data, dtype=self._dtype, count=length, offset=ptr)

    def __getitem__(self, idx: Union[int, slice]):
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            assert step == 1, "slices into an indexed dataset must be contiguous"
            return [self.get(i) for i in range(start, stop)]
        return self.get(int(idx))

    @staticmethod
    def exists(path: str) -> bool:
        return os.path.exists(index_file_path(path)) and os.path.exists(data_file_path(path))


class MMapIndexedDatasetBuilder:
    def __init__(self, out_file: str, dtype: Any = np.int64) -> None:
        self._file = open(out_file, "wb")
        self._dtype = np.dtype(dtype)
        self._sizes: list[int] = []
        self._doc_idx = [0]

    def add_item(self, tensor: Union[torch.Tensor, np.ndarray]) -> None:
        arr = np.asarray(tensor.numpy() if isinstance(tensor, torch.Tensor) else tensor, dtype=self._dtype)
        self._file.write(arr.tobytes(order="C"))
        self._sizes.append(int(arr.size))

    def end_document(self) -> None:
        self._doc_idx.append(len(self._sizes))

    def finalize(self, index_file: str) -> None:
        self._file.close()
        sizes = np.asarray(self._sizes, dtype=np.int32)
        pointers = np.zeros(len(sizes), dtype=np.int64)
        if len(sizes) > 1:
            np.cumsum(sizes[:-1].astype(np.int64) * self._dtype.itemsize, out=pointers[1:])
        with open(index_file, "wb") as f:
            f.write(MMAP_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", dtype_code(self._dtype)))
            f.write(struct.pack("<Q", len(sizes)))
            f.write(struct.pack("<Q", len(self._doc_idx)))
            f.write(sizes.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(self._doc_idx, dtype=np.int64).tobytes(order="C"))


def write_fixed_width_items(data_file: str, index_file: str, items: np.ndarray) -> None:
    """Write a 2-D array as an "mmap" indexed dataset with one item per row (every item its own document), without
    going through ``add_item`` row by row.  Files are written under temporary names and moved into place."""
    items = np.ascontiguousarray(items)
    n, width = items.shape
    tmp_data, tmp_index = f"{data_file}.tmp.{os.getpid()}", f"{index_file}.tmp.{os.getpid()}"
    items.tofile(tmp_data)
    with open(tmp_index, "wb") as f:
        f.write(MMAP_MAGIC)
        f.write(struct.pack("<Q", 1))
        f.write(struct.pack("<B", dtype_code(items.dtype)))
        f.write(struct.pack("<Q", n))
        f.write(struct.pack("<Q", n + 1))
        f.write(np.full(n, width, dtype=np.int32).tobytes(order="C"))
        f.write((np.arange(n, dtype=np.int64) * (width * items.dtype.itemsize)).tobytes(order="C"))
        f.write(np.arange(n + 1, dtype=np.int64).tobytes(order="C"))
    os.replace(tmp_data, data_file)
    os.replace(tmp_index, index_file)


class IndexedDataset(torch.utils.data.Dataset):
    """Reader of the "TNTIDX" layout; items are read from the data file on access."""

    def __init__(self, path: str) -> None:
        self.path = path
        with open(index_file_path(path), "rb") as f:
            assert f.read(8) == TNT_MAGIC, "index file does not match the expected format"
            assert struct.unpack("<Q", f.read(8)) == (1,)
            code, self.element_size = struct.unpack("<QQ", f.read(16))
            self.dtype = np.dtype(DTYPES[code])
            self._len, s = struct.unpack("<QQ", f.read(16))
            self.dim_offsets = np.fromfile(f, dtype=np.int64, count=self._len + 1)
            self.data_offsets = np.fromfile(f, dtype=np.int64, count=self._len + 1)
            self.sizes = np.fromfile(f, dtype=np.int64, count=s)
        self._data = np.memmap(data_file_path(path), mode="r", order="C") if os.path.getsize(data_file_path(path)) else None

    def __len__(self) -> int:
        return int(self._len)

    def size(self, index: int) -> np.ndarray:
        return self.sizes[self.dim_offsets[index]:self.dim_offsets[index + 1]]

    def __getitem__(self, idx: Union[int, slice]):
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            assert step == 1, "slices into an indexed dataset must be contiguous"
            return [self[i] for i in range(start, stop)]
        if idx < 0 or idx >= self._len:
            raise IndexError("index out of range")
        shape = tuple(int(x) for x in self.size(idx))
        count = int(self.data_offsets[idx + 1] - self.data_offsets[idx])
        arr = np.frombuffer(self._data, dtype=self.dtype, count=count,
                            offset=int(self.data_offsets[idx]) * self.element_size)
        return arr.reshape(shape)

    @staticmethod
    def exists(path: str) -> bool:
        return os.path.exists(index_file_path(path)) and os.path.exists(data_file_path(path))


class IndexedCachedDataset(IndexedDataset):
    """Same layout; kept as a separate name for configurations that ask for the "cached" implementation."""


class IndexedDatasetBuilder:
    element_sizes = {np.uint8: 1, np.int8: 1, np.int16: 2, np.int32: 4, np.int64: 8, np.float32: 4, np.float64: 8}

    def __init__(self, out_file: str, dtype: Any = np.int32) -> None:
        self.out_file = open(out_file, "wb")
        self.dtype = np.dtype(dtype)
        self.data_offsets = [0]
        self.dim_offsets = [0]
        self.sizes: list[int] = []
        self.element_size = self.dtype.itemsize

    def add_item(self, tensor: Union[torch.Tensor, np.ndarray]) -> None:
        arr = np.asarray(tensor.numpy() if isinstance(tensor, torch.Tensor) else tensor, dtype=self.dtype)
        self.out_file.write(arr.tobytes(order="C"))
        self.data_offsets.append(self.data_offsets[-1] + arr.size)
        self.sizes.extend(arr.shape)
        self.dim_offsets.append(self.dim_offsets[-1] + arr.ndim)

    def finalize(self, index_file: str) -> None:
        self.out_file.close()
        with open(index_file, "wb") as f:
            f.write(TNT_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<QQ", dtype_code(self.dtype), self.element_size))
            f.write(struct.pack("<QQ", len(self.data_offsets) - 1, len(self.sizes)))
            for a in (self.dim_offsets, self.data_offsets, self.sizes):
                f.write(np.asarray(a, dtype=np.int64).tobytes(order="C"))


def make_builder(out_file: str, impl: str = "mmap", vocab_size: Optional[int] = None):
    if impl == "mmap":
        return MMapIndexedDatasetBuilder(out_file, dtype=best_fitting_dtype(vocab_size))
    return IndexedDatasetBuilder(out_file)


def make_dataset(path: str, impl: str = "infer", skip_warmup: bool = True) -> Optional[torch.utils.data.Dataset]:
    """Open ``{path}.bin/.idx`` with the reader matching ``impl`` ("infer", "mmap", "lazy", "cached")."""
    if not IndexedDataset.exists(path):
        raise FileNotFoundError(f"dataset does not exist: {path}.bin / {path}.idx")
    if impl == "infer":
        impl = infer_dataset_impl(path) or ""
    if impl == "mmap":
        return MMapIndexedDataset(path, skip_warmup)
    if impl == "lazy":
        return IndexedDataset(path)
    if impl == "cached":
        return IndexedCachedDataset(path)
    raise ValueError(f"unknown dataset implementation for {path}: {impl!r}")


def get_indexed_dataset_(data_prefix: str, data_impl: str = "infer", skip_warmup: bool = True):
    return make_dataset(data_prefix, data_impl, skip_warmup)
