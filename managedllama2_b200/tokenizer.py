"""Host-side mirror of the reference's ``Tokenizer`` (src/Tokenizer.cs) over the C ABI, and the text-level loops of
``Transformer.Generate`` / ``Transformer.Chat`` (src/Transformer.cs:89-148) on top of a ``Transformer``."""
import ctypes
from dataclasses import dataclass

import numpy as np

from . import _lib


@dataclass
class Token:
    """src/Token.cs: the id and the text piece it decodes to."""
    id: int
    piece: str

    def __str__(self):
        return self.piece


class Tokenizer:
    """``new Tokenizer(tokenizerPath, vocabSize)``; ``Encode`` / ``Decode`` as src/Tokenizer.cs:57-171."""

    def __init__(self, tokenizerPath, vocabSize):
        self.lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self.lib.ml2_tokenizer_open(str(tokenizerPath).encode(), int(vocabSize), ctypes.byref(h)))
        self.handle = h

    def Encode(self, prompt, bos=False, eos=False):
        data = prompt.encode("utf-8", "surrogatepass") if isinstance(prompt, str) else bytes(prompt)
        cap = len(data) * 2 + 8
        out = (ctypes.c_int * cap)()
        n = ctypes.c_int(0)
        _lib.check(self.lib.ml2_tokenizer_encode(self.handle, data, 1 if bos else 0, 1 if eos else 0, out, cap, ctypes.byref(n)))
        return list(out[: n.value])

    def Decode(self, prev, token):
        buf = ctypes.create_string_buffer(4096)
        n = ctypes.c_int(0)
        _lib.check(self.lib.ml2_tokenizer_decode(self.handle, int(prev), int(token), buf, 4096, ctypes.byref(n)))
        return buf.raw[: n.value].decode("utf-8", "replace")

    def close(self):
        if getattr(self, "handle", None):
            self.lib.ml2_tokenizer_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _next_token(transformer, pos, generate, temperature, topP, rng):
    """Forward + Sampler.Sample (src/Transformer.cs:99-104, src/Sampler.cs:40-70)."""
    if temperature == 0.0 or not generate:
        transformer.Forward(pos, pos + 1, generate)
    else:
        transformer.Forward(pos, pos + 1, False)
        transformer.Sample(pos + 1, temperature, topP, float(rng.random(dtype=np.float32)))
    return transformer.read_token(pos + 1)


def Generate(transformer, tokenizer, prompt, steps, temperature=0.0, topP=0.9, seed=0):
    """Transformer.Generate (src/Transformer.cs:89-112): yields a ``Token`` per step, prompt pieces included."""
    rng = np.random.default_rng(seed)
    promptTokens = tokenizer.Encode(prompt, True)
    transformer.set_tokens(np.array(promptTokens, np.int32))
    prev = promptTokens[0]
    for pos in range(steps):
        generate = pos + 1 >= len(promptTokens)
        token = _next_token(transformer, pos, generate, temperature, topP, rng) if generate else promptTokens[pos + 1]
        if not generate:
            transformer.Forward(pos, pos + 1, False)
        if token < 3:
            break
        yield Token(token, tokenizer.Decode(prev, token))
        prev = token


def Chat(transformer, tokenizer, system_prompt, userInput, temperature=0.0, topP=0.9, seed=0, max_new_tokens=None):
    """Transformer.Chat (src/Transformer.cs:114-148): the Llama-2 chat template around every user turn. A turn ends
    when the model emits an id below 3 or the context is full, as there; ``max_new_tokens`` (not in the reference)
    ends it after that many generated tokens as well."""
    rng = np.random.default_rng(seed)
    pos, prev = 0, 0
    seq_len = transformer.config.seqLength
    for text in userInput:
        prompt = ("[INST] <<SYS>>\n%s\n<</SYS>>\n\n%s [/INST]" % (system_prompt, text)) if pos == 0 else "[INST] %s [/INST]" % text
        promptTokens = tokenizer.Encode(prompt, True, False)
        transformer.set_tokens(np.array(promptTokens, np.int32), first=pos)
        userPos = pos + len(promptTokens)
        made = 0
        while pos < seq_len:
            generate = pos + 1 >= userPos
            token = _next_token(transformer, pos, generate, temperature, topP, rng)
            if generate:
                if token < 3:
                    break
                yield Token(token, tokenizer.Decode(prev, token))
                made += 1
            prev = token
            pos += 1
            if max_new_tokens is not None and made >= max_new_tokens:
                break
        yield Token(0, "\n")
        pos += 1
