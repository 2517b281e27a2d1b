"""`residual_quantization._cuda`: the two operators of the reference's extension module
(plugins/residual_quantization/csrc/dispatch/binding.cpp:19-37), served by `residualquant_b200._cuda`."""

from residualquant_b200._cuda import attention, quantize

__all__ = ("attention", "quantize")
