from .nvfp4 import E2M1_VALUES, NVFP4Tensor, dequantize_nvfp4_weight, quantize_nvfp4_weight

__all__ = ["NVFP4Tensor", "quantize_nvfp4_weight", "dequantize_nvfp4_weight", "E2M1_VALUES"]
