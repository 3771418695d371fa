"""B200-native weight-only quantized linear (W8A16 / INT4) behind the reference's module API.

``kernels``       functional API (quantize, pack, dequantize, forward), mirrors ``engine/kernels``
``quantization``  ``Int8Linear`` / ``W4A16Linear`` modules and installers, mirrors ``engine/quantization``
``_lib``          the ctypes binding of ``lib/libb200q.so`` (``include/b200q.h``)
"""

__version__ = "0.1.0"
