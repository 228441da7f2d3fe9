"""The Export tab's ".bin" token file: the host library against the oracle and the hand-laid-out example."""
import json
import os

import numpy as np
import pytest

from gpu_bpe_b200 import buildBin, exportBin, mergeFiles, parseBin, vocabJson
from oracle import wgsl_model as M

HERE = os.path.dirname(os.path.abspath(__file__))


def example():
    with open(os.path.join(HERE, "golden", "dxft_example.json")) as f:
        return json.load(f)


def model_of(ex):
    vocab = [[i] for i in range(256)] + [[104, 105], [104, 105, 33]]
    return {"vocabSize": ex["vocabSize"], "vocab": vocab, "merges": [[104, 105, 256], [256, 33, 257]]}


def test_golden_example_bytes():
    ex = example()
    model = model_of(ex)
    want = bytes.fromhex(ex["bin_hex"])
    assert vocabJson(model).decode() == ex["json"] == M.vocab_json(model).decode()
    assert M.dxft_bytes(ex["tokens"], ex["vocabSize"], ex["json"].encode()) == want      # the oracle is pinned by the example
    assert buildBin(ex["tokens"], ex["vocabSize"], vocabJson(model)) == want             # and the library by both
    back = parseBin(want)
    assert back["vocabSize"] == 258 and back["tokens"].tolist() == ex["tokens"] and back["vocab"]["merges"] == model["merges"]
    assert mergeFiles([f.encode() for f in ex["files"]]).tobytes() == M.merge_files([f.encode() for f in ex["files"]]) == b"hi!\n\nhi?"


def test_random_round_trips_and_errors():
    rng = np.random.default_rng(5)
    for n in (0, 1, 7, 1000):
        toks = rng.integers(0, 70000, n, dtype=np.uint32)
        for js in (b"", b'{"version":1}'):
            b = buildBin(toks, 4096, js)
            assert b == M.dxft_bytes(toks.tolist(), 4096, js) and len(b) == 16 + 4 * n + len(js)
            assert parseBin(b)["tokens"].tolist() == toks.tolist()
    with pytest.raises(ValueError, match="Invalid .bin magic"):
        parseBin(b"\0" * 32)
    with pytest.raises(ValueError, match="Truncated .bin data"):
        parseBin(buildBin([1, 2, 3], 300)[:-1])
    with pytest.raises(ValueError, match="Truncated .bin data"):
        parseBin(b"DXFT")


@pytest.mark.gpu
def test_export_step_end_to_end(engine):
    """Train, compile the trie, encode two files through the GPU and write the .bin the Export tab would."""
    from gpu_bpe_b200 import BPETrainer, PreTokenizer, TrieTokenizer
    from tests.helpers import small_text
    data, _, _ = small_text(1, 21, 1 << 17)
    files = [data[: 50_000].tobytes(), data[50_000:].tobytes()]
    res = BPETrainer(engine).train(data, targetVocabSize=600, preTokenizer=PreTokenizer(normalize=False))
    tok = TrieTokenizer.fromVocab(engine, res["vocab"])
    name, blob = exportBin(tok, files, res)
    merged = M.merge_files(files)
    want_tokens = M.encode_bytes(merged, M.compile_vocab_to_trie(res["vocab"]), tok.chunkSize)
    model = {"vocabSize": res["vocabSize"], "vocab": res["vocab"], "merges": [list(map(int, m)) for m in res["merges"]]}
    assert blob == M.dxft_bytes(want_tokens, 600, M.vocab_json(model))
    assert name == f"train-v600-{len(want_tokens)}.bin"
    back = parseBin(blob)
    assert tok.decode(back["tokens"]) == merged and back["vocab"]["vocabSize"] == 600
    tok.destroy()
