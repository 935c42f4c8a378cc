"""B200-native quantized KV-cache path behind MIInfer's operator interface.

The product is the CUDA library `lib/libb200kv.so` (sources in `csrc/`, C ABI in
`include/b200kv.h`).  `miinfer_b200.kv` mirrors the reference's operator
interface in Python over that ABI; `miinfer_b200.build` compiles the library.
Importing `miinfer_b200.kv` fails if the library has not been built.
"""
__version__ = "0.1.0"
