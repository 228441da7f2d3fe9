"""The device pre-tokeniser against the host one (and the Python model on small inputs)."""
import numpy as np
import pytest

from gpu_bpe_b200 import PreTokenizer, synth
from oracle import wgsl_model as M

pytestmark = pytest.mark.gpu


def both(engine, data: bytes):
    host = PreTokenizer(normalize=False).preTokenizeBytes(data)["wordStarts"]
    dev = PreTokenizer(normalize=False, engine=engine).preTokenizeBytes(data)["wordStarts"]
    return host, dev


@pytest.mark.parametrize("kind,seed,n", [(1, 3, 1 << 20), (2, 4, 3 << 20), (5, 5, 2 << 20), (2, 6, 4095), (2, 7, 4097), (1, 8, 1)])
def test_synthetic_corpora(engine, kind, seed, n):
    data = synth.corpus(kind, seed, max(n, 64))[:n]
    # a slice may cut the last character short (allowed) but must not start inside one
    host, dev = both(engine, data.tobytes())
    assert np.array_equal(host, dev)


def test_rules_on_crafted_text(engine):
    pieces = ["don't stop", " we'll we've they're I'm he'd it's", " O’Neil can’t she’ll", " x'sy 'tis a'", "\n\nline\r\nnext  two   spaces\t tab",
              " 1234567 12 123 1234", " 3.14159 2,000,000", " ١٢٣٤٥٦٧ a1b2c3", " café naïve 你好世界 \U0001F600\U0001F601 !?",
              " 'S 'T 'RE 'Ve 'LL", " a'sb a's1 a's", " end'"]
    text = "".join(pieces) * 37
    host, dev = both(engine, text.encode())
    assert np.array_equal(host, dev)
    small = "".join(pieces).encode()
    want = M.pretokenize_bytes(small)[1]
    assert np.array_equal(PreTokenizer(normalize=False, engine=engine).preTokenizeBytes(small)["wordStarts"], np.frombuffer(want, np.uint8))


@pytest.mark.parametrize("run", [2, 3, 4, 4095, 4096, 4097, 8192, 12289, 100_000])
def test_long_digit_runs_cross_tiles(engine, run):
    """The every-third-digit split counts from the start of the run, however many 4,096-byte tiles back that is."""
    for lead in ("", "ab ", "x" * 4090, "٣" * 700 + " "):
        for digit in ("7", "٥"):     # one-byte and two-byte digits
            text = lead + digit * run + " tail " + digit * 5
            host, dev = both(engine, text.encode())
            assert np.array_equal(host, dev), (run, len(lead), digit)


def test_contractions_across_tile_edges(engine):
    for pad in range(4080, 4104):
        text = "a" * pad + "'ll be" + " b" * 10 + "x’ve" + " c"
        host, dev = both(engine, text.encode())
        assert np.array_equal(host, dev), pad


def test_random_valid_utf8(engine):
    rng = np.random.default_rng(11)
    alphabet = list("abcXYZ 019'\n\t.,-$") + ["’", "é", "Ж", "中", "٤", "\U0001F642", "　", " "]
    for n in (10, 1000, 50_000):
        text = "".join(rng.choice(alphabet, n))
        host, dev = both(engine, text.encode())
        assert np.array_equal(host, dev)


def test_malformed_input_is_refused(engine):
    pt = PreTokenizer(normalize=False, engine=engine)
    for bad in (b"\x80abc", b"ab\xc3", b"ab\xc3(", b"a\xe2\x80b", b"ok\xff", b"x\x80y"):
        data = bad if bad != b"ab\xc3" else None
        if data is None:
            # a character cut short at the very end is allowed
            assert np.array_equal(pt.preTokenizeBytes(b"ab\xc3")["wordStarts"], PreTokenizer(normalize=False).preTokenizeBytes(b"ab\xc3")["wordStarts"])
            continue
        with pytest.raises(Exception, match="well-formed UTF-8"):
            pt.preTokenizeBytes(data * 3)
