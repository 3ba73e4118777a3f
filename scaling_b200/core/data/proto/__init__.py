"""Protocol-buffer messages of the text-image dataset (module path of src/scaling/core/data/proto/)."""

from . import text_image_dataset_pb2

__all__ = ["text_image_dataset_pb2"]
