"""Text-level host loops (Transformer.Generate / Chat, src/Transformer.cs:89-148) over the tokenizer and the decode path."""
import numpy as np
import pytest

from test_tokenizer_cpu import base_pieces, write_tokenizer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    import managedllama2_b200 as ml2
    from managedllama2_b200.tokenizer import Tokenizer
    pieces = base_pieces() + [" "] + [chr(c) for c in range(0x21, 0x7F)] + [" a", " b", "ab", " ab", "IN", "ST", "INST", " [", "/I"]
    while len(pieces) < 512:
        pieces.append("<fill%d>" % len(pieces))
    scores = [float(len(p)) if not p.startswith("<") else -1e9 for p in pieces]
    path = tmp_path_factory.mktemp("txt") / "tokenizer.bin"
    write_tokenizer(path, pieces, scores)
    cfg = ml2.Config(dim=256, hiddenDim=384, numLayers=2, numHeads=2, numKVHeads=2, vocabSize=512, seqLength=96)
    ctx = ml2.CudaContext(0)
    tr = ml2.Transformer(cfg, ml2.synthetic_weights(ctx, cfg, seed=3, sigma=1.0), ctx)
    yield ml2, tr, Tokenizer(path, 512), pieces
    assert ctx.status() == (0, 0)
    tr.close()


def test_generate_yields_prompt_then_greedy_tokens(setup):
    ml2, tr, tok, pieces = setup
    from managedllama2_b200.tokenizer import Generate
    prompt = "ab [/INST] a"
    ids = tok.Encode(prompt, True)
    out = list(Generate(tr, tok, prompt, 24))
    want = tr.Generate(ids, 24)                       # the id-level loop of the library
    assert [t.id for t in out] == want
    assert [t.id for t in out[: len(ids) - 1]] == ids[1:]
    text = "".join(str(t) for t in out[: len(ids) - 1])
    assert text == prompt                              # the dummy prefix is stripped after BOS
    again = list(Generate(tr, tok, prompt, 24))
    assert [t.id for t in again] == [t.id for t in out]


def test_generate_with_sampling_is_reproducible(setup):
    ml2, tr, tok, pieces = setup
    from managedllama2_b200.tokenizer import Generate
    a = [t.id for t in Generate(tr, tok, "a b", 20, temperature=0.8, topP=0.9, seed=4)]
    b = [t.id for t in Generate(tr, tok, "a b", 20, temperature=0.8, topP=0.9, seed=4)]
    assert a == b and all(0 <= t < 512 for t in a)


def test_chat_turns(setup):
    ml2, tr, tok, pieces = setup
    from managedllama2_b200.tokenizer import Chat
    turns = ["ab", "a b"]
    out = list(Chat(tr, tok, "ab", turns, max_new_tokens=6))
    ends = [i for i, t in enumerate(out) if t.id == 0 and t.piece == "\n"]
    assert len(ends) == 2 and ends[-1] == len(out) - 1      # one end marker per turn (src/Transformer.cs:144)
    assert all(t.id >= 3 for i, t in enumerate(out) if i not in ends)
    assert [t.id for t in out] == [t.id for t in Chat(tr, tok, "ab", turns, max_new_tokens=6)]
