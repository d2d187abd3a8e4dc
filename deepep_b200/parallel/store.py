"""Host collectives over a ``torch.distributed`` TCPStore, for callers that have no ProcessGroup.

Parity: ``deep_ep/_store.py:16-169`` of the reference (``StoreGroup``:
sequence-numbered ``all_gather`` of JSON values, ``barrier``, chunked
``reduce_sum``, ``abort`` that wakes blocked peers, ``close``).  All ranks
must call the operations in the same order.
"""
from __future__ import annotations

import json
import os
import time
import uuid
from datetime import timedelta
from typing import Any, List

_CHUNK = 256 * 1024


class StoreAborted(RuntimeError):
    pass


class StoreGroup:
    _sessions_opened = 0          # groups this process has opened with from_env

    def __init__(self, store, rank: int, size: int, *, prefix: str, timeout: float = 300):
        if not 0 <= rank < size <= 128 or not prefix or timeout <= 0:
            raise ValueError("StoreGroup requires rank in [0, size), size <= 128, a prefix and a positive timeout")
        self._store, self._rank, self._size = store, rank, size
        self._prefix, self._timeout = prefix.rstrip("/") + "/", float(timeout)
        self._sequence = 0
        self._closed = False

    @classmethod
    def from_env(cls, timeout: float = 300, prefix: str = "deepep") -> "StoreGroup":
        """Connect to the TCPStore that torchrun already serves on MASTER_ADDR:MASTER_PORT."""
        from torch.distributed import TCPStore

        rank, size = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        store = TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), None, False,
                         timedelta(seconds=timeout))
        # one session per call: the n-th group of a process meets the n-th group of its peers (construction is
        # collective and ordered), so a second group never picks up the first one's session name
        cls._sessions_opened += 1
        key = f"{prefix}/session/" + os.environ.get("TORCHELASTIC_RESTART_COUNT", "0") + f"/{cls._sessions_opened}"
        if rank == 0:
            store.set(key, uuid.uuid4().hex)
        session = store.get(key).decode("ascii")
        group = cls(store, rank, size, prefix=f"{prefix}/{session}", timeout=timeout)
        group.barrier("connect")
        return group

    def rank(self) -> int:
        return self._rank

    def size(self) -> int:
        return self._size

    # ------------------------------------------------------------------ plumbing
    def _key(self, stage: str, who: int) -> str:
        return f"{self._prefix}{self._sequence}/{stage}/{who}"

    def abort(self, error: Any) -> None:
        """Publish a failure so that peers blocked in any operation raise instead of waiting."""
        self._store.set(self._prefix + "abort", json.dumps({"rank": self._rank, "error": str(error)}))

    def _check_abort(self) -> None:
        if self._store.check([self._prefix + "abort"]):
            info = json.loads(self._store.get(self._prefix + "abort").decode())
            raise StoreAborted(f"rank {info['rank']} aborted the group: {info['error']}")

    def _wait_get(self, key: str) -> bytes:
        deadline = time.monotonic() + self._timeout
        while True:
            if self._store.check([key]):
                return self._store.get(key)
            self._check_abort()
            if time.monotonic() > deadline:
                raise TimeoutError(f"store key {key} did not appear within {self._timeout:.0f} s")
            time.sleep(0.002)

    def _begin(self) -> None:
        if self._closed:
            raise RuntimeError("StoreGroup is closed")
        self._check_abort()
        self._sequence += 1

    # ------------------------------------------------------------------ collectives
    def all_gather(self, value: Any, stage: str = "gather") -> List[Any]:
        self._begin()
        self._store.set(self._key(stage, self._rank), json.dumps(value))
        return [json.loads(self._wait_get(self._key(stage, r)).decode()) for r in range(self._size)]

    def all_gather_bytes(self, value: bytes, stage: str = "bytes") -> List[bytes]:
        self._begin()
        self._store.set(self._key(stage, self._rank), value)
        return [bytes(self._wait_get(self._key(stage, r))) for r in range(self._size)]

    def barrier(self, stage: str = "barrier") -> None:
        self.all_gather(None, stage)

    def reduce_sum(self, array, dst: int = 0, stage: str = "reduce"):
        """Element-wise sum of equal-length int/float lists; every rank gets the result."""
        import numpy as np

        arr = np.asarray(array)
        self._begin()
        raw = arr.tobytes()
        chunks = [raw[i:i + _CHUNK] for i in range(0, max(len(raw), 1), _CHUNK)]
        self._store.set(self._key(stage, self._rank) + "/n", str(len(chunks)))
        for i, c in enumerate(chunks):
            self._store.set(self._key(stage, self._rank) + f"/{i}", c)
        total = np.zeros_like(arr)
        for r in range(self._size):
            n = int(self._wait_get(self._key(stage, r) + "/n"))
            data = b"".join(bytes(self._wait_get(self._key(stage, r) + f"/{i}")) for i in range(n))
            total = total + np.frombuffer(data, dtype=arr.dtype).reshape(arr.shape)
        del dst
        return total

    def close(self) -> None:
        if not self._closed:
            try:
                self.barrier("close")
            finally:
                self._closed = True
