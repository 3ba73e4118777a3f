"""Memory map of protobuf records, used for text + image examples (src/scaling/core/data/pb_memory_map.py:15-477,
message definitions of src/scaling/core/data/proto/text_image_dataset.proto).

Files: ``{prefix}.bin`` holds the serialised messages back to back, ``{prefix}.idx`` one ``[byte offset, byte length]``
pair per record, ``{prefix}.meta.json`` the index dtype and record count.  The message classes are built at import
time from a descriptor written in code (wire-compatible with the .proto above), so no generated module is needed:

    message PromptImageLocation { int32 start_index = 1; int32 end_index = 2; }
    message TextImageExample {
      repeated int32 input_token_list = 1; repeated int32 target_token_list = 2; repeated bool loss_mask_list = 3;
      repeated bytes prompt_image_data = 4; repeated PromptImageLocation prompt_image_locations = 5; }
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Iterable, Iterator, Optional, Type

import numpy as np
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
from google.protobuf.descriptor import FieldDescriptor
from google.protobuf.message import Message


def _build_messages() -> tuple[Type[Message], Type[Message]]:
    F = descriptor_pb2.FieldDescriptorProto
    fd = descriptor_pb2.FileDescriptorProto(name="sb200_text_image_dataset.proto", syntax="proto3")
    loc = fd.message_type.add(name="PromptImageLocation")
    loc.field.add(name="start_index", number=1, type=F.TYPE_INT32, label=F.LABEL_OPTIONAL)
    loc.field.add(name="end_index", number=2, type=F.TYPE_INT32, label=F.LABEL_OPTIONAL)
    ex = fd.message_type.add(name="TextImageExample")
    ex.field.add(name="input_token_list", number=1, type=F.TYPE_INT32, label=F.LABEL_REPEATED)
    ex.field.add(name="target_token_list", number=2, type=F.TYPE_INT32, label=F.LABEL_REPEATED)
    ex.field.add(name="loss_mask_list", number=3, type=F.TYPE_BOOL, label=F.LABEL_REPEATED)
    ex.field.add(name="prompt_image_data", number=4, type=F.TYPE_BYTES, label=F.LABEL_REPEATED)
    ex.field.add(name="prompt_image_locations", number=5, type=F.TYPE_MESSAGE, label=F.LABEL_REPEATED,
                 type_name=".PromptImageLocation")
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    get = getattr(message_factory, "GetMessageClass", None)
    if get is None:  # older protobuf
        factory = message_factory.MessageFactory(pool)
        get = factory.GetPrototype
    return get(pool.FindMessageTypeByName("PromptImageLocation")), get(pool.FindMessageTypeByName("TextImageExample"))


PromptImageLocation, TextImageExample = _build_messages()


def _is_repeated(field: FieldDescriptor) -> bool:
    flag = getattr(field, "is_repeated", None)  # newer protobuf releases; `label` is deprecated there
    if flag is None:
        return field.label == FieldDescriptor.LABEL_REPEATED
    return bool(flag() if callable(flag) else flag)


def dict2pb(message: Message, data: dict) -> Message:
    """Fill ``message`` from a (nested) dict whose keys are field names."""
    for field in message.DESCRIPTOR.fields:
        if field.name not in data:
            continue
        value = data[field.name]
        target = getattr(message, field.name)
        repeated = _is_repeated(field)
        if field.type == FieldDescriptor.TYPE_MESSAGE:
            if repeated:
                for item in value:
                    dict2pb(target.add(), item)
            else:
                dict2pb(target, value)
        elif repeated:
            target.extend(value)
        else:
            setattr(message, field.name, value)
    return message


def pb2dict(message: Message) -> dict:
    out: dict[str, Any] = {}
    for field in message.DESCRIPTOR.fields:
        value = getattr(message, field.name)
        repeated = _is_repeated(field)
        if field.type == FieldDescriptor.TYPE_MESSAGE:
            out[field.name] = [pb2dict(v) for v in value] if repeated else pb2dict(value)
        else:
            out[field.name] = list(value) if repeated else value
    return out


class PbMemoryMap:
    """Random access to the records of a protobuf memory map; ``map[i]`` is the i-th record as a dict."""

    def __init__(self, prefix_path: Path, pb_datatype: Type[Message] = TextImageExample,
                 load_index_to_memory: bool = False, initialize: bool = True):
        self.prefix_path = Path(prefix_path)
        self.pb_datatype = pb_datatype
        self.load_index_to_memory = load_index_to_memory
        self._index: Any = None
        self._data: Any = None
        self._document_count = 0
        self._index_dtype: Optional[np.dtype] = None
        if initialize:
            self.initialize()

    # the two converters as methods too (src/scaling/core/data/pb_memory_map.py:249-300 has them on the class)
    def dict2pb(self, pb_message: Message, data: dict) -> Message:
        return dict2pb(pb_message, data)

    def pb2dict(self, pb_message: Message) -> dict:
        return pb2dict(pb_message)

    @property
    def file_path_data(self) -> Path:
        return Path(str(self.prefix_path) + ".bin")

    @property
    def file_path_index(self) -> Path:
        return Path(str(self.prefix_path) + ".idx")

    @property
    def file_path_meta(self) -> Path:
        return Path(str(self.prefix_path) + ".meta.json")

    @property
    def index_dtype(self) -> Optional[np.dtype]:
        return self._index_dtype

    @property
    def document_count(self) -> int:
        return self._document_count

    def initialize(self) -> None:
        for f in (self.file_path_data, self.file_path_index, self.file_path_meta):
            if not f.is_file():
                raise FileNotFoundError(f"memory map file missing: {f}")
        with open(self.file_path_meta, "r", encoding="UTF-8") as fh:
            meta = json.load(fh)
        self._index_dtype = np.dtype(meta["index_dtype"])
        self._document_count = int(meta["document_count"])
        shape = (self._document_count, 2)
        if self.load_index_to_memory:
            self._index = np.fromfile(self.file_path_index, dtype=self._index_dtype).reshape(shape)
        else:
            self._index = np.memmap(self.file_path_index, mode="r", order="C", dtype=self._index_dtype, shape=shape)
        self._data = np.memmap(self.file_path_data, mode="r", order="C", dtype=np.uint8)

    def size(self, indices: Iterable[int]) -> list[int]:
        """Serialised size in bytes of the given records."""
        return [int(self._index[i][1]) for i in indices]

    def __len__(self) -> int:
        return self._document_count

    def __getitem__(self, index: int) -> dict:
        if index < 0 or index >= self._document_count:
            raise IndexError(f"record {index} out of range ({self._document_count} records)")
        start, length = (int(x) for x in self._index[index])
        message = self.pb_datatype()
        message.ParseFromString(bytes(self._data[start:start + length]))
        return pb2dict(message)

    def __iter__(self) -> Iterator[dict]:
        for i in range(len(self)):
            yield self[i]

    def close(self) -> None:
        self._index = None
        self._data = None


class PbMemoryMapBuilder:
    """Append-only writer.  ``add`` takes one example as a list of ``{"type": "text" | "image", "content": ...,
    "has_loss": bool}`` elements (text is tokenised, an image contributes its file bytes and placeholder tokens);
    ``add_record`` takes an already assembled record dict."""

    def __init__(self, prefix_path: Path, pb_datatype: Type[Message] = TextImageExample, tokenizer: Any = None,
                 tokenizer_no_prefix_space: Any = None, image_encoder_token_counts: int = 144,
                 index_dtype: Any = np.int64):
        self.prefix_path = Path(prefix_path)
        self.pb_datatype = pb_datatype
        self.tokenizer = tokenizer
        self.tokenizer_no_prefix_space = tokenizer_no_prefix_space
        self.image_encoder_token_counts = image_encoder_token_counts
        self.index_dtype = np.dtype(index_dtype)
        self.memory_map = PbMemoryMap(prefix_path=prefix_path, pb_datatype=pb_datatype, initialize=False)
        if self.memory_map.file_path_data.is_file():
            raise ValueError(f"data file already exists: {self.memory_map.file_path_data}")
        if self.memory_map.file_path_index.is_file():
            raise ValueError(f"index file already exists: {self.memory_map.file_path_index}")
        self.memory_map.file_path_data.parent.mkdir(exist_ok=True, parents=True)
        self.data_file = open(self.memory_map.file_path_data, "wb")
        self.index_file = open(self.memory_map.file_path_index, "wb")
        self.current_index = 0
        self.document_count = 0

    def _preprocess(self, data: list) -> dict[str, Any]:
        assert self.tokenizer is not None and self.tokenizer_no_prefix_space is not None, "tokenizers are required"
        tokens: list[int] = []
        mask: list[bool] = []
        images: list[bytes] = []
        locations: list[dict] = []
        tok = self.tokenizer_no_prefix_space  # the first text piece; later pieces use the regular tokenizer
        for item in data:
            if item["type"] == "text":
                piece = tok.encode(item["content"])
                tok = self.tokenizer
                has_loss = bool(item.get("has_loss", False))
            elif item["type"] == "image":
                piece = [self.tokenizer.padding_token_id] * self.image_encoder_token_counts
                locations.append({"start_index": len(tokens), "end_index": len(tokens) + len(piece)})
                with open(item["content"], "rb") as f:
                    images.append(f.read())
                has_loss = False
            else:
                raise NotImplementedError(f"Content type {item['type']} is not supported")
            tokens.extend(piece)
            mask.extend([has_loss] * len(piece))
        return {"input_token_list": tokens[:-1], "target_token_list": tokens[1:], "loss_mask_list": mask[1:],
                "prompt_image_data": images, "prompt_image_locations": locations}

    def add_record(self, record: dict) -> None:
        serialized = dict2pb(self.pb_datatype(), record).SerializeToString()
        self.data_file.write(serialized)
        self.index_file.write(np.array([self.current_index, len(serialized)]).astype(self.index_dtype).tobytes(order="C"))
        self.current_index += len(serialized)
        self.document_count += 1

    def add(self, data: list) -> None:
        self.add_record(self._preprocess(data))

    def finalize(self) -> None:
        self.data_file.close()
        self.index_file.close()
        with open(self.memory_map.file_path_meta, "w", encoding="UTF-8") as f:
            json.dump({"index_dtype": self.index_dtype.name, "document_count": self.document_count}, f)

    def __del__(self) -> None:
        for name in ("data_file", "index_file"):
            f = getattr(self, name, None)
            if f is not None and not f.closed:
                f.close()
