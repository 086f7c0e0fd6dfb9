"""Liveness of the ranks of one job: a heartbeat word per rank, checked on the host before a step is launched.

A rank that dies (or leaves) between steps must not leave the others waiting inside their next collective or peer
wait until a long process-group timeout: every rank bumps its own word in a small shared table a few times a second,
and before launching a step a rank looks at the others' words.  A word that has not moved for ``timeout_s`` means the
rank is gone; a rank that leaves on purpose says so.  ``check()`` then raises ``RankLostError`` naming the ranks, and
the caller can stop cleanly (save what it has, tear the group down) while its own GPU work is still in order.

The reference has no such mechanism: its ranks rely on the 100 s process-group timeout
(src/executable/perf_emb.py:169-173) and an experiment-level watchdog (src/kg/scripts/exp_config.py:119-139).

Two carriers for the table:

* ``backend="shm"``: a named shared-memory tensor (``ipc.IPCTensorFactory``); ranks are processes of one box.
* ``backend="store"``: the keys ``{name}/{rank}`` of a ``torch.distributed`` store (TCPStore / FileStore), for ranks
  that share no memory.

The table must be fresh for a job (a word left over from an earlier job would read as a rank that has left): use a
name or shared-memory namespace of the job's own, or clear the shared memory at start-up as the drivers do.

Staleness is judged by the observer's own monotonic clock (it remembers when it last saw a word change), so the
ranks need no common clock.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

import torch

ALIVE, LEFT = 1, 2


class RankLostError(RuntimeError):
    """One or more ranks stopped beating (``lost``) or announced that they leave (``left``)."""

    def __init__(self, lost: List[int], left: List[int], timeout_s: float):
        parts = []
        if lost:
            parts.append(f"rank(s) {lost} gave no sign of life for {timeout_s:g} s")
        if left:
            parts.append(f"rank(s) {left} left the job")
        super().__init__("; ".join(parts))
        self.lost, self.left = lost, left


class Heartbeat:
    def __init__(self, rank: int, world: int, name: str = "rs_heartbeat", period_s: float = 0.1, backend: str = "shm",
                 store=None):
        assert 0 <= rank < world
        assert backend in ("shm", "store")
        self.rank, self.world, self.name, self.period_s, self.backend = rank, world, name, float(period_s), backend
        self._store = store
        if backend == "store":
            assert store is not None, "backend='store' needs a torch.distributed store"
            self._table = None
        else:
            from ..ipc import IPCTensorFactory
            # [rank] = (beat counter, state, barrier generation)
            self._table = IPCTensorFactory.NewOrGetIPCTensor(name, (world, 3), torch.int64)
        self._gen = 0
        self._write_gen(0)
        self._write(0, 0)                            # nothing of an earlier owner of this row survives
        self._seen: Dict[int, tuple] = {}            # rank -> (last counter value, local time it changed)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._beats = 0

    # ---------------------------------------------------------------- my own word
    def _write(self, beats: int, state: int) -> None:
        if self._table is not None:
            self._table[self.rank, 1] = state
            self._table[self.rank, 0] = beats
        else:
            self._store.set(f"{self.name}/{self.rank}", f"{beats} {state}")

    def _write_gen(self, gen: int) -> None:
        if self._table is not None:
            self._table[self.rank, 2] = gen
        else:
            self._store.set(f"{self.name}/{self.rank}/gen", str(gen))

    def _read_gen(self, r: int) -> int:
        if self._table is not None:
            return int(self._table[r, 2])
        try:
            k = f"{self.name}/{r}/gen"
            return int(self._store.get(k).decode()) if self._store.check([k]) else 0
        except Exception:
            return -1

    def beat(self) -> None:
        """One sign of life (the background thread calls this; a caller without the thread may call it per step)."""
        self._beats += 1
        self._write(self._beats, ALIVE)

    def start(self) -> "Heartbeat":
        if self._thread is None:
            self.beat()
            self._stop.clear()

            def run():
                while not self._stop.wait(self.period_s):
                    try:
                        self.beat()
                    except Exception:            # the carrier is gone (the rank that hosted the store has exited):
                        return                   # nothing left to tell anybody
            self._thread = threading.Thread(target=run, name=f"heartbeat-{self.rank}", daemon=True)
            self._thread.start()
        return self

    def stop(self, leaving: bool = True) -> None:
        """Stops beating; ``leaving`` tells the others at once that this rank is gone on purpose."""
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None
        if leaving:
            self._beats += 1
            self._write(self._beats, LEFT)

    # ---------------------------------------------------------------- the others' words
    def _read(self, r: int):
        if self._table is not None:
            row = self._table[r]
            return int(row[0]), int(row[1])
        try:
            if not self._store.check([f"{self.name}/{r}"]):
                return 0, 0
            b, s = self._store.get(f"{self.name}/{r}").decode().split()
            return int(b), int(s)
        except Exception:                      # the store itself is gone: whoever hosted it has died
            return -1, 0

    def status(self, timeout_s: float) -> Dict[str, List[int]]:
        """``{"lost": [...], "left": [...], "unseen": [...]}`` among the other ranks.  ``unseen``: never beat yet (still
        starting); they count as lost once ``timeout_s`` has passed since this observer first looked."""
        now = time.monotonic()
        lost, left, unseen = [], [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            beats, state = self._read(r)
            prev = self._seen.get(r)
            if prev is None or prev[0] != beats:
                self._seen[r] = (beats, now)
                prev = self._seen[r]
            if state == LEFT:
                left.append(r)
            elif now - prev[1] > timeout_s:
                lost.append(r)
            elif beats == 0:
                unseen.append(r)
        return {"lost": lost, "left": left, "unseen": unseen}

    def check(self, timeout_s: float = 2.0) -> None:
        """Raises ``RankLostError`` when another rank is gone; call it on the host before every launch."""
        st = self.status(timeout_s)
        if st["lost"] or st["left"]:
            raise RankLostError(st["lost"], st["left"], timeout_s)

    def wait_all_alive(self, timeout_s: float = 30.0) -> None:
        """Blocks until every rank has beaten at least once (start-up rendezvous)."""
        t0 = time.monotonic()
        while True:
            st = self.status(timeout_s)
            if st["left"] or st["lost"]:
                raise RankLostError(st["lost"], st["left"], timeout_s)
            if not st["unseen"]:
                return
            if time.monotonic() - t0 > timeout_s:
                raise RankLostError(st["unseen"], [], timeout_s)
            time.sleep(min(0.02, self.period_s))

    def barrier(self, timeout_s: float = 2.0, poll_s: float = 0.005) -> None:
        """A host barrier of all ranks that cannot hang on a dead rank: returns when every rank has entered its
        barrier of the same count (or a later one), raises ``RankLostError`` as soon as one of them is found gone."""
        self._gen += 1
        self._write_gen(self._gen)
        others = [r for r in range(self.world) if r != self.rank]
        while True:
            if all(self._read_gen(r) >= self._gen for r in others):
                return
            self.check(timeout_s)
            time.sleep(poll_s)

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop(leaving=True)
