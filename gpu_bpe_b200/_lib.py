"""ctypes binding of libb200bpe.so (the C ABI of include/b200bpe.h).

There is no fallback: if the shared library is missing, or no sm_100 GPU is visible when a
context is created, the call raises.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libb200bpe.so")
SYNTH_PATH = os.path.join(PKG, "libb200bpe_synth.so")

u8p, u32p, u64p = C.POINTER(C.c_uint8), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)

COMPAT_LITERAL, COMPAT_FIXED = 0, 1
FLAG_NO_GRAPH, FLAG_TIME_KERNELS, FLAG_FULL_RECOUNT, FLAG_NCCL_EXCHANGE = 1, 2, 4, 8

STATUS = {0: "OK", 1: "BAD_ARG", 2: "CUDA", 3: "NO_DEVICE", 4: "EMPTY_CORPUS", 5: "TABLE_FULL", 6: "LOOKBACK_TIMEOUT",
          7: "BAD_TRIE_MAGIC", 8: "BAD_TRIE_VERSION", 9: "TRUNCATED_TRIE", 10: "CAPACITY", 11: "NCCL", 12: "OOM",
          13: "INTERNAL"}


class TrainOpts(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("target_vocab_size", C.c_uint32), ("first_token_id", C.c_uint32),
                ("batch_merges", C.c_uint32), ("compat_mode", C.c_uint32), ("table_log2", C.c_uint32),
                ("flags", C.c_uint32), ("exchange_cap", C.c_uint32), ("test_lookback_spins", C.c_uint32),
                ("test_first_tile", C.c_uint32)]


class TokOpts(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("chunk_size", C.c_uint32), ("layout", C.c_uint32), ("test_lookback_spins", C.c_uint32),
                ("batch_slice_bytes", C.c_uint64), ("encode_slice_bytes", C.c_uint64)]


TRIE_LAYOUTS = {"auto": 0, "cuckoo": 1, "hybrid": 2, "hash": 3}


class Progress(C.Structure):
    _fields_ = [("merge_index", C.c_uint32), ("total_merges", C.c_uint32), ("last_a", C.c_uint32),
                ("last_b", C.c_uint32), ("last_new_id", C.c_uint32), ("last_count", C.c_uint32),
                ("symbol_count", C.c_uint64), ("merges_per_second", C.c_double)]


class KernelStats(C.Structure):
    _fields_ = [("pair_count_ms", C.c_double), ("argmax_ms", C.c_double), ("merge_compact_ms", C.c_double),
                ("exchange_ms", C.c_double), ("pair_count_launches", C.c_uint64), ("argmax_launches", C.c_uint64),
                ("merge_compact_launches", C.c_uint64), ("exchange_launches", C.c_uint64),
                ("pair_count_bytes", C.c_uint64), ("argmax_bytes", C.c_uint64), ("merge_compact_bytes", C.c_uint64),
                ("pair_count_skipped_ms", C.c_double), ("pair_count_skipped_launches", C.c_uint64),
                ("table_update_ms", C.c_double)]


PROGRESS_CB = C.CFUNCTYPE(None, C.POINTER(Progress), C.c_void_p)

# name → (restype, argtypes); also the list of symbols the header declares
SIGNATURES = {
    "b200bpe_status_str": (C.c_char_p, [C.c_int32]),
    "b200bpe_last_error": (C.c_char_p, []),
    "b200bpe_device_count": (C.c_int32, []),
    "b200bpe_ctx_create": (C.c_int32, [C.c_int32, C.POINTER(C.c_void_p)]),
    "b200bpe_nccl_unique_id": (C.c_int32, [C.c_char_p, u8p]),
    "b200bpe_ctx_create_dist": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_char_p, u8p, C.POINTER(C.c_void_p)]),
    "b200bpe_ctx_destroy": (None, [C.c_void_p]),
    "b200bpe_ctx_info": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), u64p, u64p]),
    "b200bpe_ctx_synchronize": (C.c_int32, [C.c_void_p]),
    "b200bpe_train": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(TrainOpts), u32p, u32p, u32p,
                                  u32p, PROGRESS_CB, C.c_void_p]),
    "b200bpe_trainer_create": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(TrainOpts),
                                           C.POINTER(C.c_void_p)]),
    "b200bpe_trainer_create_device": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(TrainOpts),
                                                  C.POINTER(C.c_void_p)]),
    "b200bpe_trainer_create_from_symbols": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(TrainOpts),
                                                        C.POINTER(C.c_void_p)]),
    "b200bpe_trainer_run": (C.c_int32, [C.c_void_p, C.c_uint32, u32p, u32p, u32p, u32p, PROGRESS_CB, C.c_void_p]),
    "b200bpe_trainer_reset": (C.c_int32, [C.c_void_p]),
    "b200bpe_trainer_symbols": (C.c_int32, [C.c_void_p, u32p, C.c_uint64, u64p]),
    "b200bpe_trainer_pair_counts": (C.c_int32, [C.c_void_p, u64p, u32p, C.c_uint64, u64p]),
    "b200bpe_trainer_kernel_stats": (C.c_int32, [C.c_void_p, C.POINTER(KernelStats)]),
    "b200bpe_trainer_last_run_ms": (C.c_int32, [C.c_void_p, C.POINTER(C.c_double)]),
    "b200bpe_trainer_last_reset_ms": (C.c_int32, [C.c_void_p, C.POINTER(C.c_double)]),
    "b200bpe_trainer_launches": (C.c_int32, [C.c_void_p, u64p]),
    "b200bpe_trainer_exchange_kind": (C.c_int32, [C.c_void_p, u32p]),
    "b200bpe_trainer_destroy": (None, [C.c_void_p]),
    "b200bpe_trie_compile": (C.c_int32, [C.c_void_p, u64p, C.c_uint32, C.c_void_p, C.POINTER(C.c_size_t)]),
    "b200bpe_trie_parse_header": (C.c_int32, [C.c_void_p, C.c_size_t, u32p]),
    "b200bpe_tokenizer_create": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint32, C.POINTER(C.c_void_p)]),
    "b200bpe_tokenizer_create_ex": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(TokOpts), C.POINTER(C.c_void_p)]),
    "b200bpe_tokenizer_info": (C.c_int32, [C.c_void_p, u32p, u32p, u32p, u32p]),
    "b200bpe_tokenizer_layout": (C.c_int32, [C.c_void_p, u32p, u32p]),
    "b200bpe_encode": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, u64p]),
    "b200bpe_encode_batch": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64,
                                         C.c_void_p]),
    "b200bpe_encode_device": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, u64p]),
    "b200bpe_encode_batch_device": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p,
                                                C.c_uint64, C.c_void_p, u64p]),
    "b200bpe_encode_device_noalloc": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, u64p]),
    "b200bpe_tokenizer_last_ms": (C.c_int32, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "b200bpe_tokenizer_destroy": (None, [C.c_void_p]),
    "b200bpe_replay_create": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(C.c_void_p)]),
    "b200bpe_replay_encode": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, u64p]),
    "b200bpe_replay_encode_device": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, u64p]),
    "b200bpe_replay_last_rounds": (C.c_int32, [C.c_void_p, u32p]),
    "b200bpe_replay_destroy": (None, [C.c_void_p]),
    "b200bpe_pretokenize": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "b200bpe_pretokenize_device": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]),
    "b200bpe_pretokenize_device_ex": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint32]),
    "b200bpe_pretokenize_gpu": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]),
    "b200bpe_dxft_size": (C.c_int32, [C.c_uint64, C.c_uint64, u64p]),
    "b200bpe_dxft_write": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "b200bpe_dxft_parse": (C.c_int32, [C.c_void_p, C.c_uint64, u32p, u64p, u64p]),
}

_lib = None
_synth = None


class B200BPEError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
        self.status_name = STATUS.get(status, str(status))


def lib():
    """Load libb200bpe.so; raises if it has not been built (python -m gpu_bpe_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} is missing: build it with `python -m gpu_bpe_b200.build`; "
                                    "there is no CPU fallback")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def synth():
    global _synth
    if _synth is None:
        S = C.CDLL(SYNTH_PATH)
        S.b200bpe_synth_corpus.argtypes = [C.c_int, C.c_uint64, C.c_uint64, C.c_void_p, C.c_int]
        S.b200bpe_synth_corpus.restype = C.c_int
        S.b200bpe_synth_corpus_range.argtypes = [C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_int]
        S.b200bpe_synth_corpus_range.restype = C.c_int
        S.b200bpe_synth_doc_offsets.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_double, C.c_void_p]
        S.b200bpe_synth_doc_offsets.restype = C.c_int
        _synth = S
    return _synth


def check(status: int, what: str = ""):
    if status != 0:
        L = lib()
        msg = L.b200bpe_status_str(status).decode()
        detail = L.b200bpe_last_error().decode()
        raise B200BPEError(status, f"{what + ': ' if what else ''}{msg}" + (f" ({detail})" if detail and status in (2, 3, 11, 12) else ""))


def nccl_library_path() -> str:
    """Path of the NCCL that PyTorch ships, so the process holds one NCCL only."""
    try:
        import nvidia.nccl as _n  # type: ignore
        for base in list(_n.__path__):
            p = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(p):
                return p
    except Exception:
        pass
    return "libnccl.so.2"
