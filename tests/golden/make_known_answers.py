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

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "known_answers.json")
    with open(out, "w") as f:
        json.dump({"word_start_marker": "|", "cases": CASES}, f, indent=1)
    print(out)
