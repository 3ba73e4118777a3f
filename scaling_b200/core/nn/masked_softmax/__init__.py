from .masked_softmax import MaskedSoftmax, MaskedSoftmaxConfig, MaskedSoftmaxKernel

__all__ = ["MaskedSoftmax", "MaskedSoftmaxConfig", "MaskedSoftmaxKernel"]
