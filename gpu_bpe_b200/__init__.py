"""gpu_bpe_b200 — B200-native BPE training and trie encoding behind the API of toprakdeviren/gpu-bpe.

The compute path is libb200bpe.so (hand-written CUDA for sm_100a, C ABI in include/b200bpe.h);
these modules are the host-side mirror of the reference's JavaScript classes.
"""
from .engine import BPEEngine
from .export import buildBin, exportBin, mergeFiles, parseBin, vocabJson
from .pretokenizer import PreTokenizer
from .tokenizer import TrieTokenizer
from .trainer import BPETrainer, TrainerSession
from .trie import compileVocabToTrie, parseHeader, parseTrieBuffers
from .vocab import Vocab, model_from_json, model_to_json

__all__ = ["BPEEngine", "BPETrainer", "TrainerSession", "TrieTokenizer", "PreTokenizer", "Vocab", "compileVocabToTrie",
           "parseHeader", "parseTrieBuffers", "model_to_json", "model_from_json", "mergeFiles", "vocabJson", "buildBin",
           "parseBin", "exportBin"]
