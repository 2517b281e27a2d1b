"""B200-native (sm_100a) packed-KV kernels: the KV-write quantizer and the packed paged decode attention of
ResidualQuant-style KV-cache compression for looped Transformers, behind the reference's operator API.

    from residualquant_b200 import _cuda            # attention(...), quantize(...): reference signatures
    from residualquant_b200.rotation import register_rotation
"""

__version__ = "0.1.0"
