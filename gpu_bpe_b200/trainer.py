"""BPETrainer — BPE vocabulary training on a B200.

Mirrors BPETrainer of src/bpe/trainer.js:125-371 of the reference: the same constructor, the
same train(input, {targetVocabSize, preTokenizer, onProgress}) arguments and result object, the
same error for an empty corpus, the same progress payload.  The merge loop itself runs in
libb200bpe.so (128 merges per CUDA-graph launch, one read-back per batch).
"""
from __future__ import annotations

import ctypes as C
import time

import numpy as np

from . import _lib
from .vocab import Vocab

BATCH_SIZE = 128  # training-pipeline.js:13


def _format_duration(seconds: float) -> str:  # trainer.js:31-36
    if seconds < 60:
        return f"{seconds:.1f}s"
    m, s = int(seconds // 60), round(seconds % 60)
    return f"{m}m {s}s" if s > 0 else f"{m}m"


def prepare_input(data, preTokenizer):
    """prepareInput (trainer.js:62-107) → (bytes u8 array, word-start mask or None)."""
    if preTokenizer is not None and not isinstance(data, str):
        arr = np.frombuffer(bytes(data), np.uint8) if not isinstance(data, np.ndarray) else data
        r = preTokenizer.preTokenizeBytes(arr)
        if r["bytes"].size == 0 and arr.size > 0:
            return arr, None
        return r["bytes"], r["wordStarts"]
    if preTokenizer is not None and isinstance(data, str):
        r = preTokenizer.preTokenize(data)
        if r["bytes"].size == 0 and len(data) > 0:
            return np.frombuffer(data.encode("utf-8"), np.uint8), None
        return r["bytes"], r["wordStarts"]
    raw = data.encode("utf-8") if isinstance(data, str) else data
    arr = np.frombuffer(bytes(raw), np.uint8) if not isinstance(raw, np.ndarray) else np.ascontiguousarray(raw, np.uint8)
    return arr, None


class TrainerSession:
    """A corpus resident on the device: run merges, reset, inspect.  Thin wrapper of b200bpe_trainer_*."""

    def __init__(self, engine, handle, merges_goal: int):
        self.engine, self._h, self.merges_goal = engine, handle, merges_goal
        self._keep = []

    @staticmethod
    def _opts(target_vocab_size, first_token_id, compat_mode, batch_merges, table_log2, flags, exchange_cap=0,
              test_lookback_spins=0, test_first_tile=0):
        o = _lib.TrainOpts()
        o.exchange_cap = exchange_cap
        o.test_lookback_spins, o.test_first_tile = test_lookback_spins, test_first_tile
        o.struct_size = C.sizeof(_lib.TrainOpts)
        o.target_vocab_size, o.first_token_id = target_vocab_size, first_token_id
        o.batch_merges, o.table_log2, o.flags = batch_merges, table_log2, flags
        o.compat_mode = {"literal": _lib.COMPAT_LITERAL, "fixed": _lib.COMPAT_FIXED}[compat_mode]
        return o

    @classmethod
    def create(cls, engine, data: np.ndarray, word_starts, *, target_vocab_size=4096, first_token_id=256,
               compat_mode="literal", batch_merges=BATCH_SIZE, table_log2=0, flags=0, device_pointers=False,
               n: int | None = None, exchange_cap=0, test_lookback_spins=0, test_first_tile=0):
        o = cls._opts(target_vocab_size, first_token_id, compat_mode, batch_merges, table_log2, flags, exchange_cap,
                      test_lookback_spins, test_first_tile)
        h = C.c_void_p()
        L = _lib.lib()
        if device_pointers:
            st = L.b200bpe_trainer_create_device(engine.ctx, C.c_void_p(int(data)),
                                                 C.c_void_p(int(word_starts)) if word_starts else None, n, C.byref(o),
                                                 C.byref(h))
        else:
            data = np.ascontiguousarray(data, np.uint8)
            ws = None if word_starts is None else np.ascontiguousarray(word_starts, np.uint8)
            st = L.b200bpe_trainer_create(engine.ctx, data.ctypes.data if data.size else None,
                                          ws.ctypes.data if ws is not None and ws.size else None, data.size, C.byref(o),
                                          C.byref(h))
        _lib.check(st, "b200bpe_trainer_create")
        return cls(engine, h, target_vocab_size - first_token_id)

    @classmethod
    def from_symbols(cls, engine, symbols: np.ndarray, **kw):
        o = cls._opts(kw.get("target_vocab_size", 4096), kw.get("first_token_id", 256), kw.get("compat_mode", "literal"),
                      kw.get("batch_merges", BATCH_SIZE), kw.get("table_log2", 0), kw.get("flags", 0), 0,
                      kw.get("test_lookback_spins", 0), kw.get("test_first_tile", 0))
        sym = np.ascontiguousarray(symbols, np.uint32)
        h = C.c_void_p()
        _lib.check(_lib.lib().b200bpe_trainer_create_from_symbols(engine.ctx, sym.ctypes.data if sym.size else None,
                                                                 sym.size, C.byref(o), C.byref(h)),
                   "b200bpe_trainer_create_from_symbols")
        return cls(engine, h, o.target_vocab_size - o.first_token_id)

    def run(self, max_merges: int = 0, on_progress=None):
        """→ (merges (M,3) u32 [a, b, new_id], counts (M,) u32, early_stop)."""
        cap = max(1, self.merges_goal)
        merges = np.zeros((cap, 3), np.uint32)
        counts = np.zeros(cap, np.uint32)
        n, es = C.c_uint32(), C.c_uint32()
        cb = _lib.PROGRESS_CB(lambda p, _u: on_progress(p.contents)) if on_progress else _lib.PROGRESS_CB()
        st = _lib.lib().b200bpe_trainer_run(self._h, max_merges, merges.ctypes.data_as(_lib.u32p),
                                            counts.ctypes.data_as(_lib.u32p), C.byref(n), C.byref(es), cb, None)
        _lib.check(st, "b200bpe_trainer_run")
        return merges[: n.value].copy(), counts[: n.value].copy(), bool(es.value)

    def reset(self):
        _lib.check(_lib.lib().b200bpe_trainer_reset(self._h), "b200bpe_trainer_reset")

    def symbols(self) -> np.ndarray:
        n = C.c_uint64()
        _lib.check(_lib.lib().b200bpe_trainer_symbols(self._h, None, 0, C.byref(n)))
        out = np.zeros(max(1, n.value), np.uint32)
        _lib.check(_lib.lib().b200bpe_trainer_symbols(self._h, out.ctypes.data_as(_lib.u32p), out.size, C.byref(n)))
        return out[: n.value]

    def pair_counts(self, cap: int = 1 << 22) -> dict[int, int]:
        keys, cnts, n = np.zeros(cap, np.uint64), np.zeros(cap, np.uint32), C.c_uint64()
        _lib.check(_lib.lib().b200bpe_trainer_pair_counts(self._h, keys.ctypes.data_as(_lib.u64p),
                                                         cnts.ctypes.data_as(_lib.u32p), cap, C.byref(n)))
        return dict(zip(keys[: n.value].tolist(), cnts[: n.value].tolist()))

    def kernel_stats(self) -> dict:
        ks = _lib.KernelStats()
        _lib.check(_lib.lib().b200bpe_trainer_kernel_stats(self._h, C.byref(ks)))
        return {f: getattr(ks, f) for f, _ in _lib.KernelStats._fields_}

    def launches(self) -> int:
        """Kernel launches of this trainer since it was created (a graph launch counts its kernels)."""
        n = C.c_uint64()
        _lib.check(_lib.lib().b200bpe_trainer_launches(self._h, C.byref(n)))
        return n.value

    def exchange_kind(self) -> str:
        """'none' (one GPU), 'peer' (this library's kernels over NVLink peer memory) or 'nccl'."""
        k = C.c_uint32()
        _lib.check(_lib.lib().b200bpe_trainer_exchange_kind(self._h, C.byref(k)))
        return ("none", "peer", "nccl")[k.value]

    def last_run_ms(self) -> float:
        ms = C.c_double()
        _lib.check(_lib.lib().b200bpe_trainer_last_run_ms(self._h, C.byref(ms)))
        return ms.value

    def last_reset_ms(self) -> float:
        ms = C.c_double()
        _lib.check(_lib.lib().b200bpe_trainer_last_reset_ms(self._h, C.byref(ms)))
        return ms.value

    def destroy(self):
        if self._h is not None:
            _lib.lib().b200bpe_trainer_destroy(self._h)
            self._h = None


class BPETrainer:
    def __init__(self, engine, compat_mode: str | None = None):
        self._engine = engine
        self._vocab = Vocab()
        # "literal" reproduces the reference as shipped; sharded jobs need "fixed"
        self.compat_mode = compat_mode or ("literal" if getattr(engine, "world", 1) == 1 else "fixed")

    def train(self, input, targetVocabSize: int = 4096, preTokenizer=None, onProgress=None) -> dict:
        data, word_starts = prepare_input(input, preTokenizer)
        if data.size == 0 and self._engine.world == 1:
            raise ValueError("No symbols to train on — corpus is empty after pre-processing")  # trainer.js:161-163
        merges_needed = targetVocabSize - self._vocab.size  # trainer.js:208
        merges: list[list[int]] = []
        if merges_needed <= 0:
            return self._result(merges, 0.0)
        first_id = self._vocab.nextTokenId
        o = TrainerSession._opts(first_id + merges_needed, first_id, self.compat_mode, BATCH_SIZE, 0, 0)
        out = np.zeros((merges_needed, 3), np.uint32)
        n, es = C.c_uint32(), C.c_uint32()
        vocab = self._vocab

        # The progress payload needs the merged string, so the vocabulary is extended per batch
        # inside the callback path: entries for ids below last_new_id are added lazily.
        seen = [0]

        def _cb_wrap(p, u):
            pc = p.contents
            while seen[0] < pc.merge_index:
                a, b, _nid = (int(x) for x in out[seen[0]])
                vocab.addMerge(a, b)
                merges.append([a, b, _nid])
                seen[0] += 1
            if onProgress:
                onProgress({"mergeIndex": pc.merge_index, "totalMerges": pc.total_merges,
                            "mergeString": vocab.strings[-1] if pc.last_count else "—",
                            "bestCount": pc.last_count, "symbolCount": pc.symbol_count,
                            "mergesPerSecond": pc.merges_per_second})

        cb = _lib.PROGRESS_CB(_cb_wrap)
        t0 = time.perf_counter()
        ws = None if word_starts is None else np.ascontiguousarray(word_starts, np.uint8)
        data = np.ascontiguousarray(data, np.uint8)
        st = _lib.lib().b200bpe_train(self._engine.ctx, data.ctypes.data if data.size else None,
                                      ws.ctypes.data if ws is not None and ws.size else None, data.size, C.byref(o),
                                      out.ctypes.data_as(_lib.u32p), None, C.byref(n), C.byref(es), cb, None)
        _lib.check(st, "b200bpe_train")
        while seen[0] < n.value:
            a, b, nid = (int(x) for x in out[seen[0]])
            vocab.addMerge(a, b)
            merges.append([a, b, nid])
            seen[0] += 1
        self.earlyStop = bool(es.value)
        return self._result(merges, time.perf_counter() - t0)

    def _result(self, merges, seconds):
        return {"vocab": self._vocab.entries, "vocabStrings": self._vocab.strings, "vocabSize": self._vocab.size,
                "merges": merges, "trainingTime": _format_duration(seconds)}

    def exportVocab(self) -> str:
        return self._vocab.export()
