from .decoder import Decoder, Layer, tensor_requests

__all__ = ["Decoder", "Layer", "tensor_requests"]
