"""Host-side mirror of the reference's operator classes over the C ABI.

Each class keeps the name, constructor arguments and ``Forward`` argument meaning of the C# class it
stands for (src/<Name>.cs of GilesBathgate/ManagedLlama2); device buffers are torch CUDA tensors
(fp16 / int32 / uint32-as-int32) instead of ``CudaDeviceVariable``. Launch geometry is decided
inside the library, so the constructors only keep what ``Forward`` needs.
"""
import ctypes
from dataclasses import dataclass

from . import _lib


def ceil_div(a, b):
    return (a + (b - 1)) // b


def qweight_sizes(rows):
    """(weightsSize, zerosSize, scalesSize) per output row, src/QKVMatVec.cs:22-24."""
    scales = ceil_div(rows, 128)
    return ceil_div(rows, 32) * 4, ceil_div(scales, 8), scales


@dataclass
class Config:
    """src/Config.cs:6-17 (same field order as the 32-byte file header)."""
    dim: int
    hiddenDim: int
    numLayers: int
    numHeads: int
    numKVHeads: int
    vocabSize: int
    seqLength: int
    ropeTheta: float = 10000.0

    def to_struct(self):
        return _lib.ConfigStruct(self.dim, self.hiddenDim, self.numLayers, self.numHeads, self.numKVHeads,
                                 self.vocabSize, self.seqLength, self.ropeTheta)


class CudaContext:
    """Stands for ManagedCuda's ``CudaContext(deviceID)`` (src/Transformer.cs:48-49)."""

    def __init__(self, deviceID=0):
        self._lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self._lib.ml2_ctx_create(ctypes.c_int(deviceID), ctypes.byref(h)))
        self.handle = h
        self.device = deviceID

    def set_stream(self, stream_ptr):
        _lib.check(self._lib.ml2_ctx_set_stream(self.handle, ctypes.c_void_p(stream_ptr)))

    def set_pdl(self, enabled):
        _lib.check(self._lib.ml2_ctx_set_pdl(self.handle, ctypes.c_int(1 if enabled else 0)))

    def synchronize(self):
        _lib.check(self._lib.ml2_ctx_synchronize(self.handle))

    def set_wait_limit(self, sm_cycles):
        """Budget of every device-side wait, in SM clock cycles (default 2e10, about ten seconds)."""
        _lib.check(self._lib.ml2_ctx_set_wait_limit(self.handle, ctypes.c_longlong(int(sm_cycles))))

    def status(self):
        err, det = ctypes.c_uint(), ctypes.c_uint()
        _lib.check(self._lib.ml2_ctx_status(self.handle, ctypes.byref(err), ctypes.byref(det)))
        return err.value, det.value

    @property
    def launch_count(self):
        return int(self._lib.ml2_ctx_launch_count(self.handle))

    def close(self):
        if self.handle:
            self._lib.ml2_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _ptr(t, offset_elems=0):
    """Device pointer of a torch tensor, optionally offset by elements (OffsetPointer, src/Extensions.cs:20-21)."""
    return ctypes.c_void_p(t.data_ptr() + offset_elems * t.element_size())


class QWeight:
    """src/QWeight.cs:5-10: Weight (uint32), Zeros (uint32), Scales (fp16) device arrays."""

    def __init__(self, Weight, Zeros, Scales):
        self.Weight, self.Zeros, self.Scales = Weight, Zeros, Scales

    def struct(self):
        return _lib.QWeightStruct(self.Weight.data_ptr(), self.Zeros.data_ptr(), self.Scales.data_ptr())


class Module:
    """src/Module.cs:7-26. The PTX-per-module loading is replaced by the shared library."""

    def __init__(self, cudaContext):
        self.ctx = cudaContext
        self.lib = cudaContext._lib

    @staticmethod
    def CeilDiv(a, b):
        return ceil_div(a, b)


class MatVec(Module):
    """src/MatVec.cs:6-17."""

    def __init__(self, cudaContext, config=None):
        super().__init__(cudaContext)

    def Forward(self, output, input, matrix, rows, cols):
        _lib.check(self.lib.ml2_matvec_f16(self.ctx.handle, _ptr(output), _ptr(input), _ptr(matrix), rows, cols))


class QKVMatVec(Module):
    """src/QKVMatVec.cs:7-32."""

    def __init__(self, cudaContext, config):
        super().__init__(cudaContext)
        self.kvDim = config.dim * config.numKVHeads // config.numHeads

    def Forward(self, queryOutput, keyOutput, valueOutput, input, query, key, value, rows, cols, layerOffset, pos):
        offset = layerOffset + pos * self.kvDim  # :25
        q, k, v = query.struct(), key.struct(), value.struct()
        _lib.check(self.lib.ml2_qkv_matvec_int4(self.ctx.handle, _ptr(queryOutput), _ptr(keyOutput, offset),
                                                _ptr(valueOutput, offset), _ptr(input), ctypes.byref(q),
                                                ctypes.byref(k), ctypes.byref(v), rows, cols))


class MatVecSwiGLU(Module):
    """src/MatVecSwiGLU.cs:6-24."""

    def __init__(self, cudaContext, config=None):
        super().__init__(cudaContext)

    def Forward(self, output, input, g, u, rows, cols):
        gs, us = g.struct(), u.struct()
        _lib.check(self.lib.ml2_matvec_swiglu_int4(self.ctx.handle, _ptr(output), _ptr(input), ctypes.byref(gs),
                                                   ctypes.byref(us), rows, cols))


class MatVecResidual(Module):
    """src/MatVecResidual.cs:6-24."""

    def __init__(self, cudaContext, config=None):
        super().__init__(cudaContext)

    def Forward(self, output, input, matrix, rows, cols):
        m = matrix.struct()
        _lib.check(self.lib.ml2_matvec_residual_int4(self.ctx.handle, _ptr(output), _ptr(input), ctypes.byref(m), rows,
                                                     cols))


class MatVecStrided(Module):
    """src/MatVecStrided.cs:7-19. ``seqLength`` is the live length (pos + 1)."""

    def __init__(self, cudaContext, config):
        super().__init__(cudaContext)
        self.numHeads = config.numHeads

    def Forward(self, attention, query, key, headSize, dim, seqLength, layerOffset, scale):
        _lib.check(self.lib.ml2_matvec_strided(self.ctx.handle, _ptr(attention), _ptr(query), _ptr(key, layerOffset),
                                               headSize, dim, self.numHeads, seqLength, ctypes.c_float(scale)))


class VecMat(Module):
    """src/VecMat.cs:7-19."""

    def __init__(self, cudaContext, config):
        super().__init__(cudaContext)
        self.numHeads = config.numHeads

    def Forward(self, output, value, attention, headSize, dim, seqLength, layerOffset):
        _lib.check(self.lib.ml2_vecmat(self.ctx.handle, _ptr(output), _ptr(value, layerOffset), _ptr(attention),
                                       headSize, dim, self.numHeads, seqLength))


class RMSNorm(Module):
    """src/RMSNorm.cs:5-15."""

    def Forward(self, output, input, weights, size, eps=1e-5):
        _lib.check(self.lib.ml2_rmsnorm(self.ctx.handle, _ptr(output), _ptr(input), _ptr(weights), size,
                                        ctypes.c_float(eps)))


class RoPERotation(Module):
    """src/RoPERotation.cs:6-24."""

    def __init__(self, cudaContext, config):
        super().__init__(cudaContext)
        self.kvDim = config.dim * config.numKVHeads // config.numHeads
        self.numHeads = config.numHeads

    def Forward(self, query, key, numKVHeads, headSize, pos, layerOffset, theta):
        offset = layerOffset + pos * self.kvDim  # :22
        _lib.check(self.lib.ml2_rope(self.ctx.handle, _ptr(query), _ptr(key, offset), self.numHeads, numKVHeads,
                                     headSize, pos, ctypes.c_float(theta)))


class Softmax(Module):
    """src/Softmax.cs:5-15."""

    def __init__(self, cudaContext, config):
        super().__init__(cudaContext)
        self.numHeads = config.numHeads

    def Forward(self, attention, seqLength):
        _lib.check(self.lib.ml2_softmax(self.ctx.handle, _ptr(attention), self.numHeads, seqLength))


class Embedding(Module):
    """src/Embedding.cs:5-15."""

    def __init__(self, cudaContext, config=None):
        super().__init__(cudaContext)

    def Forward(self, output, table, size, tokens, pos):
        _lib.check(self.lib.ml2_embedding(self.ctx.handle, _ptr(output), _ptr(table), size, _ptr(tokens), pos))


class Argmax(Module):
    """src/Argmax.cs:5-15."""

    def Forward(self, logits, vocabSize, tokens, nextPos, generateToken):
        _lib.check(self.lib.ml2_argmax(self.ctx.handle, _ptr(logits), vocabSize, _ptr(tokens), nextPos,
                                       1 if generateToken else 0))


class SoftmaxLogits(Module):
    """src/SoftmaxLogits.cs:5-16."""

    def Forward(self, logits, size, temperature, indices):
        _lib.check(self.lib.ml2_softmax_logits(self.ctx.handle, _ptr(logits), size, ctypes.c_float(temperature), _ptr(indices)))


class Sort(Module):
    """src/Sort.cs:5-16 (descending by key, values carried; any size up to 32768)."""

    def __init__(self, cudaContext, config=None):
        super().__init__(cudaContext)

    def Forward(self, logits, indices, size):
        _lib.check(self.lib.ml2_sort(self.ctx.handle, _ptr(logits), _ptr(indices), size))


class CumulativeSum(Module):
    """src/CumulativeSum.cs:5-16."""

    def __init__(self, cudaContext, config=None):
        super().__init__(cudaContext)

    def Forward(self, logits, size):
        _lib.check(self.lib.ml2_cumulative_sum(self.ctx.handle, _ptr(logits), size))


class SampleTopP(Module):
    """src/SampleTopP.cs:5-16."""

    def Forward(self, logits, indices, size, threshold, tokens, nextPos):
        _lib.check(self.lib.ml2_sample_top_p(self.ctx.handle, _ptr(logits), _ptr(indices), size, ctypes.c_float(threshold),
                                             _ptr(tokens), nextPos))
