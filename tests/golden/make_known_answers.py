"""Writes known_answers.json: the hand-derived training cases of the merge loop.

Each case was worked out by hand from the reference's shader source (src/bpe/train.wgsl and the
dispatch order of src/bpe/training-pipeline.js:178-222); this script only stores them.  '|'
marks a word start; the first symbol is always one.  "literal" = the reference as shipped
(compaction input bounded by the post-merge count), "fixed" = compaction over every pre-merge
position.  Symbols are shown as hex words: bit 16 = word start, low 16 bits = token id.
"""
import json
import os

CASES = [
    {"input": "abab",
     "literal": {"merges": [[97, 98, 256, 2]], "symbols": ["0x10100", "0x0"]},
     "fixed": {"merges": [[97, 98, 256, 2]], "symbols": ["0x10100", "0x100"]}},
    {"input": "aaaa",
     "literal": {"merges": [[97, 97, 256, 3]], "symbols": ["0x10100"]},
     "fixed": {"merges": [[97, 97, 256, 3]], "symbols": ["0x10100"]}},
    {"input": "aa|aa",
     "literal": {"merges": [[97, 97, 256, 2]], "symbols": ["0x10100", "0x0"]},
     "fixed": {"merges": [[97, 97, 256, 2]], "symbols": ["0x10100", "0x10100"]}},
    {"input": "acaaca",
     "literal": {"merges": [[97, 99, 256, 2]], "symbols": ["0x10100", "0x61", "0x100", "0x0"]},
     "fixed": {"merges": [[97, 99, 256, 2], [256, 97, 257, 2]], "symbols": ["0x10101", "0x101"]}},
    {"input": "ab| ab| ab| cab",
     "literal": {"merges": [[97, 98, 256, 4], [32, 256, 257, 2]],
                 "symbols": ["0x10100", "0x10101", "0x10101", "0x0", "0x62", "0x10020"]},
     "fixed": {"merges": [[97, 98, 256, 4], [32, 256, 257, 2]],
               "symbols": ["0x10100", "0x10101", "0x10101", "0x10020", "0x63", "0x100"]}},
    # ties: (a,b) and (c,d) both occur twice → the smaller packed pair id wins (train.wgsl:83-85)
    {"input": "cd|ab|cd|ab",
    # (literal: the second compaction leaves the stale 'b' of the first source buffer in the tail)
     "literal": {"merges": [[97, 98, 256, 2], [99, 100, 257, 2]], "symbols": ["0x10101", "0x10100", "0x10101", "0x62"]},
     "fixed": {"merges": [[97, 98, 256, 2], [99, 100, 257, 2]], "symbols": ["0x10101", "0x10100", "0x10101", "0x10100"]}},
    # a pair that only ever straddles a word start is never counted → immediate early stop
    {"input": "a|b|a|b",
     "literal": {"merges": [], "symbols": ["0x10061", "0x10062", "0x10061", "0x10062"]},
     "fixed": {"merges": [], "symbols": ["0x10061", "0x10062", "0x10061", "0x10062"]}},
]

# Merge-replay encoding (TokenizerManager.encode, src/ui/tokenizer-manager.js:13-61), worked out by hand from
# that loop: one token per byte, then every rule in learned order, each one left-to-right pass that steps over
# both tokens of a match.
REPLAY_CASES = [
    {"text": "aaa", "merges": [[97, 97, 256]], "tokens": [256, 97]},                      # pairs from the left, the odd one stays
    {"text": "aaaa", "merges": [[97, 97, 256]], "tokens": [256, 256]},                    # not one token, unlike the trainer's merge
    {"text": "aaaaa", "merges": [[97, 97, 256], [256, 256, 257]], "tokens": [257, 97]},
    {"text": "abab", "merges": [[97, 98, 256], [256, 256, 257]], "tokens": [257]},
    {"text": "abc", "merges": [[98, 99, 256], [97, 98, 257]], "tokens": [97, 256]},       # the earlier rule takes the b
    {"text": "abc", "merges": [[97, 98, 256], [98, 99, 257]], "tokens": [256, 99]},
    {"text": "xyz", "merges": [[97, 98, 256]], "tokens": [120, 121, 122]},                # no rule applies
    {"text": "", "merges": [[97, 98, 256]], "tokens": []},
    {"text": "ab", "merges": [], "tokens": [97, 98]},                                     # no merges: byte level (:21-25)
    {"text": "a b a b", "merges": [[97, 32, 256], [256, 98, 257]], "tokens": [257, 32, 257]},           # no word boundaries on this path
    {"text": "é", "merges": [[195, 169, 256]], "tokens": [256]},                          # bytes of the UTF-8 encoding
]

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "known_answers.json")
    with open(out, "w") as f:
        json.dump({"word_start_marker": "|", "cases": CASES, "replay": REPLAY_CASES}, f, indent=1, ensure_ascii=True)
    print(out)
