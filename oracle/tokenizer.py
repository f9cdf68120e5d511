"""Pure-Python restatement of the reference's Tokenizer (src/Tokenizer.cs:27-171), UTF-16 semantics included: strings
are lists of UTF-16 code units, ordinal comparison is on those units, Encode walks code units, and StrLookup treats a
hit at index 0 of the sorted vocabulary as a miss (`i > 0`, :92). Test infrastructure (the checker of
``ml2_tokenizer_*``); the reference's own golden vectors (test/TransformerTests.cs:25-33) need the real Llama-2
``tokenizer.bin``, which is not available offline, so only their structure (byte fallback, dummy prefix, BOS / EOS
pieces) is reproduced by the tests: parity unpinned."""
import bisect
import re
import struct

BOS, EOS = 1, 2


def u16(s):
    """str -> tuple of UTF-16 code units (lone surrogates pass through)."""
    b = s.encode("utf-16-le", "surrogatepass")
    return tuple(struct.unpack("<%dH" % (len(b) // 2), b))


def from_u16(units):
    return struct.pack("<%dH" % len(units), *units).decode("utf-16-le", "replace")


def utf8_lenient(data):
    return bytes(data).decode("utf-8", "replace")


class Tokenizer:
    def __init__(self, path, vocab_size):
        with open(path, "rb") as f:
            (self.max_token_length,) = struct.unpack("<i", f.read(4))
            self.vocab, self.scores = [], []
            for _ in range(vocab_size):
                score, n = struct.unpack("<fi", f.read(8))
                self.vocab.append(u16(utf8_lenient(f.read(n))))
                self.scores.append(score)
        self.sorted = sorted((s, i) for i, s in enumerate(self.vocab))     # ordinal on code units; ties by id
        self.keys = [s for s, _ in self.sorted]
        self.multibyte = []

    def lookup(self, units):
        i = bisect.bisect_left(self.keys, units)
        if i == len(self.keys) or self.keys[i] != units:
            return -1
        return self.sorted[i][1] if i > 0 else -1

    def encode(self, prompt, bos=False, eos=False):
        p = u16(prompt)
        tokens = [BOS] if bos else []
        if p:
            tokens.append(self.lookup(u16(" ")))
        prev = 0
        for c in p:
            tid = self.lookup((c,))
            if tid != -1:
                tokens.append(tid)
                continue
            if 0xD800 <= c <= 0xDBFF:
                prev = c
                continue
            chars = (prev, c) if (0xD800 <= prev <= 0xDBFF and 0xDC00 <= c <= 0xDFFF) else (c,)
            tokens.extend(b + 3 for b in from_u16(chars).encode("utf-8"))
            prev = 0
        while True:
            best, best_id, best_idx = float("-inf"), -1, -1
            for i in range(len(tokens) - 1):
                tid = self.lookup(self.vocab[tokens[i]] + self.vocab[tokens[i + 1]])
                if tid != -1 and self.scores[tid] > best:
                    best, best_id, best_idx = self.scores[tid], tid, i
            if best_idx == -1:
                break
            tokens[best_idx] = best_id
            del tokens[best_idx + 1]
        if eos:
            tokens.append(EOS)
        return tokens

    _white = set(list(range(9, 14)) + [0x20, 0x85, 0xA0, 0x1680] + list(range(0x2000, 0x200B)) + [0x2028, 0x2029, 0x202F, 0x205F, 0x3000])

    def decode(self, prev, token):
        piece = list(self.vocab[token])
        if prev == BOS and piece[0] == 0x20:
            while piece and piece[0] in self._white:
                piece.pop(0)
        text = from_u16(piece)
        m = re.match(r"^<0x([0-9A-F]{2})>$", text)
        if m:
            value = int(m.group(1), 16)
            self.multibyte.append(value)
            if value > 0x80 or (value & 0xC0) == 0x80:
                return ""
        if not self.multibyte:
            return text
        result = utf8_lenient(self.multibyte)
        if not m:
            result += text
        self.multibyte = []
        return result
