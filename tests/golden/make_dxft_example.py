"""Writes dxft_example.json: a hand-laid-out ".bin" token file (src/ui/export-controller.js:235-248).

The bytes were written down by hand from the format (four little-endian u32 header words: magic
0x44584654, vocabSize, tokenCount, vocabJsonBytes; the tokens as little-endian u32; the JSON text);
this script only stores them, as hex, next to the inputs that must produce them."""
import json
import os

MODEL = {"vocabSize": 258, "vocab_tail": [[104, 105], [104, 105, 33]], "merges": [[104, 105, 256], [256, 33, 257]]}
JSON_TEXT = ('{"version":1,"vocabSize":258,"vocab":[' + ",".join(f"[{i}]" for i in range(256)) +
             ',[104,105],[104,105,33]],"merges":[[104,105,256],[256,33,257]]}')
TOKENS = [257, 10, 10, 256, 63]           # "hi!" "\n" "\n" "hi" "?"  =  files "hi!" and "hi?" joined by two line feeds
HEADER_HEX = "54465844" "02010000" "05000000"   # 'TFXD' on disk (little-endian magic), 258, 5 tokens
TOKENS_HEX = "01010000" "0a000000" "0a000000" "00010000" "3f000000"

if __name__ == "__main__":
    js = JSON_TEXT.encode("utf-8")
    length_hex = len(js).to_bytes(4, "little").hex()
    out = {"files": ["hi!", "hi?"], "tokens": TOKENS, "vocabSize": 258, "json": JSON_TEXT,
           "bin_hex": HEADER_HEX + length_hex + TOKENS_HEX + js.hex(), "name": "train-v258-5.bin"}
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "dxft_example.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote dxft_example.json:", 16 + 20 + len(js), "bytes of .bin")
