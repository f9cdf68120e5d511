"""Tokenizer through the C ABI against the pure-Python restatement, on synthetic ``tokenizer.bin`` files in the
reference's format. The structure of the reference's golden cases (test/TransformerTests.cs:25-33) is reproduced:
token 1 = "\\n<s>\\n", 2 = "\\n</s>\\n", 3..258 the <0xNN> byte pieces, " " at id 29871 of 32000, so that "\\n" must
encode to [1, 29871, 13, 2] and the llama emoji to [1, 29871, 243, 162, 169, 156, 2] exactly as there; the word-level
cases depend on the real vocabulary's merges, which is not available offline."""
import struct

import numpy as np
import pytest

import managedllama2_b200 as ml2
from managedllama2_b200.tokenizer import Tokenizer
from oracle.tokenizer import Tokenizer as OracleTokenizer


def write_tokenizer(path, pieces, scores):
    with open(path, "wb") as f:
        f.write(struct.pack("<i", max(len(p.encode()) for p in pieces)))
        for p, s in zip(pieces, scores):
            b = p.encode("utf-8")
            f.write(struct.pack("<fi", s, len(b)))
            f.write(b)


def base_pieces():
    return ["<unk>", "\n<s>\n", "\n</s>\n"] + ["<0x%02X>" % b for b in range(256)]


@pytest.fixture(scope="module")
def llama_like(tmp_path_factory):
    """32000 pieces: specials, bytes, filler, single characters, and merge chains for a few words."""
    pieces = base_pieces()
    scores = [0.0] * len(pieces)
    words = [" You", " are", " a", " helpful", " assistant", " <<", "SY", ">>", " [", "INST", "SYS", "ST", "IN"]
    chain = []
    for w in words:                       # every prefix of a word is a piece, longer = better score
        for k in range(2, len(w) + 1):
            if w[:k] not in chain:
                chain.append(w[:k])
    singles = [chr(c) for c in range(0x21, 0x7F)] + ["é", "ß", "中", "文"]
    body = chain + singles
    while len(pieces) + len(body) < 29871:
        pieces.append("<filler%d>" % len(pieces))
        scores.append(-1e9)
    for i, p in enumerate(body[: 29871 - len(pieces)] if len(pieces) + len(body) > 29871 else body):
        pieces.append(p)
        scores.append(float(len(p)) - i * 1e-4)
    while len(pieces) < 29871:
        pieces.append("<pad%d>" % len(pieces))
        scores.append(-1e9)
    pieces.append(" ")                    # id 29871
    scores.append(-1.0)
    while len(pieces) < 32000:
        pieces.append("<tail%d>" % len(pieces))
        scores.append(-1e9)
    path = tmp_path_factory.mktemp("tok") / "tokenizer.bin"
    write_tokenizer(path, pieces, scores)
    return path, pieces


def test_golden_structure_cases(llama_like):
    path, pieces = llama_like
    tok = Tokenizer(path, 32000)
    assert pieces[29871] == " "
    assert tok.Encode("\n", True, True) == [1, 29871, 13, 2]                       # test/TransformerTests.cs:30
    assert tok.Encode("\U0001F999", True, True) == [1, 29871, 243, 162, 169, 156, 2]   # :31
    assert tok.Encode("", True, True) == [1, 2]
    # decode loop of Test_TokenizerDecode (:47-62)
    for text, ids in (("\n", [1, 29871, 13, 2]), ("\U0001F999", [1, 29871, 243, 162, 169, 156, 2])):
        out, prev = "", 0
        for t in ids:
            out += tok.Decode(prev, t)
            prev = t
        assert out == "\n<s>\n" + text + "\n</s>\n"


def test_words_merge_to_single_pieces(llama_like):
    path, pieces = llama_like
    tok = Tokenizer(path, 32000)
    ids = tok.Encode("You are a helpful assistant", True, True)
    assert [pieces[i] for i in ids[1:-1]] == [" You", " are", " a", " helpful", " assistant"]
    assert [pieces[i] for i in tok.Encode("[/INST]", True, True)[1:-1]] == [" [", "/", "INST", "]"]


@pytest.mark.parametrize("seed", range(6))
def test_against_python_restatement(llama_like, tmp_path, seed):
    rng = np.random.default_rng(seed)
    if seed < 3:
        path, pieces = llama_like
        vocab = 32000
    else:
        # a small random vocabulary with random scores: merges compete, ties and the index-0 quirk occur
        alphabet = list("abcde \n") + ["é", "中"]
        pieces = base_pieces() + [" "] + alphabet
        for _ in range(120):
            k = int(rng.integers(2, 5))
            p = "".join(rng.choice(alphabet, k))
            if p not in pieces:
                pieces.append(p)
        scores = [float(s) for s in rng.integers(-5, 6, len(pieces))]
        path = tmp_path / "tok.bin"
        write_tokenizer(path, pieces, scores)
        vocab = len(pieces)
    tok, ref = Tokenizer(path, vocab), OracleTokenizer(path, vocab)
    chars = list("abcde  \n[]/<>INSTYouarehlpfi") + ["é", "中", "文", "ß", "\U0001F999", "\u2003", "x\u0301"]
    for _ in range(60):
        text = "".join(rng.choice(chars, int(rng.integers(0, 24))))
        bos, eos = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        ids = tok.Encode(text, bos, eos)
        assert ids == ref.encode(text, bos, eos), text
        got, want, prev = "", "", 0
        for t in ids:
            got += tok.Decode(prev, t)
            want += ref.decode(prev, t)
            prev = t
        assert got == want, text


def test_text_survives_a_round_trip(llama_like):
    path, _ = llama_like
    tok = Tokenizer(path, 32000)
    for text in ("You are a helpful assistant", "a é 中文 \U0001F999 ok", "[INST] <<SYS>>\nhi\n<</SYS>>\n\nyo [/INST]"):
        ids = tok.Encode(text, True, False)
        out, prev = "", 0
        for t in ids + [tok.Encode("!", False, False)[-1]]:   # a plain piece at the end flushes pending bytes
            out += tok.Decode(prev, t)
            prev = t
        assert out == "\n<s>\n" + text + "!"


def test_errors(tmp_path, llama_like):
    path, _ = llama_like
    with pytest.raises(ml2.Ml2Error):
        Tokenizer(tmp_path / "missing.bin", 10)
    with pytest.raises(ml2.Ml2Error):
        Tokenizer(path, 40000)                     # more pieces asked for than the file holds
    tok = Tokenizer(path, 32000)
    with pytest.raises(ml2.Ml2Error):
        tok.Decode(0, 32000)
