"""Import alias: the reference's plugin package name.

The reference's vLLM hook does `from residual_quantization._cuda import attention, quantize`
(plugins/residual_quantization/src/residual_quantization/packed_backend.py:17-20, install_cache.py:195).  With this
directory on the path that line resolves to the sm_100a kernels of `residualquant_b200` unchanged.
"""
