"""AWQ checkpoint -> ``model.bin``: host-side mirror of the reference's ``ModelConverter`` (src/ModelConverter.cs).

The checkpoint files are read with ``torch.load`` (the reference walks the zip archive with its own unpickler,
:177-188, :334-395), ``config.json`` gives the header (:71-122), tensors are written in the order of
``Convert`` (:130-177) and the AWQ tensors are re-packed on the GPU by the library
(``ml2_awq_repack_qdata`` / ``ml2_awq_repack_scales`` / ``ml2_awq_compact_scales_v1``; RepackQWeightByName, :196-284).
There is no download step (the reference's ``Downloader`` classes): paths of local files are required.
"""
import ctypes
import json
import struct

import numpy as np

from . import _lib
from .modules import Config, CudaContext, ceil_div

GROUP = 128


def load_config(configPath):
    """JsonConfig.Convert (src/ModelConverter.cs:100-121)."""
    with open(configPath) as f:
        j = json.load(f)
    theta = j.get("rope_theta")
    return Config(dim=j["hidden_size"], hiddenDim=j["intermediate_size"], numLayers=j["num_hidden_layers"],
                  numHeads=j["num_attention_heads"], numKVHeads=j["num_key_value_heads"], vocabSize=j["vocab_size"],
                  seqLength=j["max_position_embeddings"], ropeTheta=10000.0 if theta is None else float(theta))


class ModelConverter:
    """``new ModelConverter(modelPath, configPath, modelType, download: false)`` + ``Convert(outputPath, format)``."""

    def __init__(self, modelPaths, configPath, cudaContext=None, download=False):
        if download:
            raise ValueError("downloading is not available: pass the paths of local checkpoint files")
        self.modelPaths = [modelPaths] if isinstance(modelPaths, (str, bytes)) or hasattr(modelPaths, "__fspath__") else list(modelPaths)
        self.configPath = configPath
        self.ctx = cudaContext or CudaContext(0)
        self.lib = self.ctx._lib

    # -- device re-packing --------------------------------------------------------------------------
    def _dev(self, t):
        import torch
        return t.contiguous().to("cuda:%d" % self.ctx.device)

    def repack_qdata(self, t, height, width):
        """RepackQData (src/ModelConverter.cs:286-321) of an int32 tensor [height][width / 8]."""
        import torch
        src = self._dev(t.view(torch.int32).reshape(-1)[: height * (width // 8)])
        out = torch.empty(width * ceil_div(height, 8), dtype=torch.int32, device=src.device)
        _lib.check(self.lib.ml2_awq_repack_qdata(self.ctx.handle, ctypes.c_void_p(src.data_ptr()), height, width,
                                                 ctypes.c_void_p(out.data_ptr())))
        self.ctx.synchronize()
        return out.cpu().numpy().view(np.uint32)

    def repack_scales(self, t, meta_height, width):
        import torch
        src = self._dev(t.reshape(-1)[: meta_height * width])
        out = torch.empty(meta_height * width, dtype=torch.float16, device=src.device)
        _lib.check(self.lib.ml2_awq_repack_scales(self.ctx.handle, ctypes.c_void_p(src.data_ptr()), meta_height, width,
                                                  ctypes.c_void_p(out.data_ptr())))
        self.ctx.synchronize()
        return out.cpu().numpy()

    def compact_scales_v1(self, t, scales_size, padded_height, width):
        import torch
        src = self._dev(t.reshape(-1)[: padded_height * width])
        out = torch.empty(scales_size * width, dtype=torch.float16, device=src.device)
        _lib.check(self.lib.ml2_awq_compact_scales_v1(self.ctx.handle, ctypes.c_void_p(src.data_ptr()), scales_size,
                                                      padded_height, width, ctypes.c_void_p(out.data_ptr())))
        self.ctx.synchronize()
        return out.cpu().numpy()

    # -- Convert ------------------------------------------------------------------------------------
    def _state(self):
        import torch
        state = {}
        for p in self.modelPaths:   # UpdateStateDictionary, src/ModelConverter.cs:177-188
            for k, v in torch.load(p, map_location="cpu", weights_only=True).items():
                if k in state:
                    raise ValueError("tensor %s appears in more than one checkpoint file" % k)
                state[k] = v
        return state

    @staticmethod
    def _half_bytes(t, name):
        import torch
        if t.dtype != torch.float16:
            raise ValueError("%s: fp16 expected, found %s (the reference copies the stored bytes as they are)" % (name, t.dtype))
        return t.contiguous().numpy().tobytes()

    def _qweight(self, out, state, prefix, height, width, fmt):
        """RepackQWeightByName (src/ModelConverter.cs:196-284): weights, zero points, scales of one projection."""
        import torch
        scales_size, zeros_size = ceil_div(height, GROUP), ceil_div(ceil_div(height, GROUP), 8)
        qw, qz, sc = state[prefix + ".qweight"], state[prefix + ".qzeros"], state[prefix + ".scales"]
        if qw.dtype != torch.int32 or qz.dtype != torch.int32 or sc.dtype != torch.float16:
            raise ValueError("%s: int32 qweight / qzeros and fp16 scales expected" % prefix)
        if fmt == "v0":
            out.write(self.repack_qdata(qw, height, width).tobytes())
            out.write(self.repack_qdata(qz, scales_size, width).tobytes())
            out.write(self.repack_scales(sc, scales_size, width).tobytes())
        elif fmt == "v1":
            out.write(qw.contiguous().numpy().tobytes()[: ceil_div(height, 8) * width * 4])
            out.write(qz.contiguous().numpy().tobytes()[: zeros_size * width * 4])
            out.write(self.compact_scales_v1(sc, scales_size, zeros_size * 8, width).tobytes())
        else:
            raise ValueError("Format is not supported")   # src/ModelConverter.cs:236, 279

    def Convert(self, outputPath, format="v0"):
        config = load_config(self.configPath)
        state = self._state()
        kv_dim = config.dim * config.numKVHeads // config.numHeads
        with open(outputPath, "wb") as out:
            out.write(struct.pack("<7if", config.dim, config.hiddenDim, config.numLayers, config.numHeads, config.numKVHeads,
                                  config.vocabSize, config.seqLength, config.ropeTheta))   # Config.SaveConfig
            for name in ("model.embed_tokens.weight", "lm_head.weight", "model.norm.weight"):
                out.write(self._half_bytes(state[name], name))
            for i in range(config.numLayers):
                L = "model.layers.%d" % i
                self._qweight(out, state, L + ".self_attn.q_proj", config.dim, config.dim, format)
                self._qweight(out, state, L + ".self_attn.k_proj", config.dim, kv_dim, format)
                self._qweight(out, state, L + ".self_attn.v_proj", config.dim, kv_dim, format)
                self._qweight(out, state, L + ".self_attn.o_proj", config.dim, config.dim, format)
                self._qweight(out, state, L + ".mlp.up_proj", config.dim, config.hiddenDim, format)
                self._qweight(out, state, L + ".mlp.gate_proj", config.dim, config.hiddenDim, format)
                self._qweight(out, state, L + ".mlp.down_proj", config.hiddenDim, config.dim, format)
                for name in (L + ".input_layernorm.weight", L + ".post_attention_layernorm.weight"):
                    out.write(self._half_bytes(state[name], name))
        return config
