from .inference_model import CompletionOutput, TransformerInferenceModule
from .sample import sample_argmax, sample_temperature, top_k_transform, top_p_transform

__all__ = ["CompletionOutput", "TransformerInferenceModule", "sample_argmax", "sample_temperature",
           "top_k_transform", "top_p_transform"]
