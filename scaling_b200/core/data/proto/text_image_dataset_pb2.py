"""``TextImageExample`` and ``PromptImageLocation`` under the name of the generated module of
src/scaling/core/data/proto/text_image_dataset_pb2.py.  The classes are built at import time from a descriptor
written out in ``pb_memory_map.py`` (no generated code, no protoc step); the wire format is the same."""

from ..pb_memory_map import PromptImageLocation, TextImageExample

__all__ = ["PromptImageLocation", "TextImageExample"]
