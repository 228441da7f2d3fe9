"""BPEEngine — the device handle the trainer and the tokenizer are built on.

Stands where src/bpe/engine.js:181-245 of the reference stands (adapter, device, compiled
pipelines); here it owns one b200bpe context: one B200, one CUDA stream.
"""
from __future__ import annotations

import ctypes as C

from . import _lib


class BPEEngine:
    def __init__(self, device: int = 0):
        self.device_index = device
        self._ctx = None
        self.rank, self.world = 0, 1

    def init(self) -> "BPEEngine":
        """Create the context.  Raises if the library or a B200 is missing (no CPU path)."""
        if self._ctx is None:
            h = C.c_void_p()
            _lib.check(_lib.lib().b200bpe_ctx_create(self.device_index, C.byref(h)), "b200bpe_ctx_create")
            self._ctx = h
        return self

    def init_distributed(self, rank: int, world: int, unique_id: bytes, nccl_lib: str | None = None) -> "BPEEngine":
        """Join a sharded job: one engine per GPU, all given the same NCCL unique id."""
        h = C.c_void_p()
        uid = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        path = (nccl_lib or _lib.nccl_library_path()).encode()
        _lib.check(_lib.lib().b200bpe_ctx_create_dist(self.device_index, rank, world, path, uid, C.byref(h)),
                   "b200bpe_ctx_create_dist")
        self._ctx, self.rank, self.world = h, rank, world
        return self

    @staticmethod
    def make_unique_id(nccl_lib: str | None = None) -> bytes:
        uid = (C.c_uint8 * 128)()
        path = (nccl_lib or _lib.nccl_library_path()).encode()
        _lib.check(_lib.lib().b200bpe_nccl_unique_id(path, uid), "b200bpe_nccl_unique_id")
        return bytes(uid)

    @property
    def ctx(self):
        if self._ctx is None:
            raise RuntimeError("BPEEngine not initialized. Call init() first.")  # engine.js:240-244
        return self._ctx

    @property
    def limits(self) -> dict:
        sm, cc, tot, free = C.c_int32(), C.c_int32(), C.c_uint64(), C.c_uint64()
        _lib.check(_lib.lib().b200bpe_ctx_info(self.ctx, C.byref(sm), C.byref(cc), C.byref(tot), C.byref(free)))
        return {"smCount": sm.value, "computeCapability": cc.value, "totalMemory": tot.value, "freeMemory": free.value}

    def synchronize(self):
        _lib.check(_lib.lib().b200bpe_ctx_synchronize(self.ctx))

    def destroy(self):
        if self._ctx is not None:
            _lib.lib().b200bpe_ctx_destroy(self._ctx)
            self._ctx = None
