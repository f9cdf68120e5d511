"""B200-native decode hot path for ManagedLlama2 (AWQ int4 group-128 mat-vec family, attention
products, RMSNorm / RoPE / softmax) behind the reference's operator API.

The compute lives in ``libml2b200.so`` (hand-written sm_100a CUDA behind the C ABI of
``include/ml2b200.h``). This package is the host-side mirror of the reference's C# classes
(``Module`` subclasses, ``QWeight``, ``Config``, ``RunState``, ``Transformer``) on top of that ABI;
PyTorch is used for device buffers and streams only.
"""
from ._lib import LIB_PATH, Ml2Error, declared_symbols, load  # noqa: F401
from .modules import (Argmax, Config, CudaContext, Embedding, MatVec, MatVecResidual, MatVecStrided,  # noqa: F401
                      MatVecSwiGLU, QKVMatVec, QWeight, RMSNorm, RoPERotation, Softmax, VecMat, ceil_div,
                      CumulativeSum, SampleTopP, SoftmaxLogits, Sort,
                      qweight_sizes)

from .transformer import (DeviceWeights, ModelFile, PerLayerWeight, Transformer, TransformerWeights, synthetic_weights,  # noqa: F401,E402
                          synthetic_weights_host, tp_shapes)

__all__ = ["DeviceWeights", "ModelFile", "PerLayerWeight", "Transformer", "TransformerWeights", "synthetic_weights", "synthetic_weights_host", "tp_shapes",
           "Argmax", "Config", "CudaContext", "Embedding", "MatVec", "MatVecResidual", "MatVecStrided",
           "MatVecSwiGLU", "QKVMatVec", "CumulativeSum", "SampleTopP", "SoftmaxLogits", "Sort", "QWeight", "RMSNorm", "RoPERotation", "Softmax", "VecMat", "Ml2Error",
           "load", "declared_symbols", "ceil_div", "qweight_sizes", "LIB_PATH"]
