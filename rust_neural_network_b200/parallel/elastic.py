"""Host-side failure detection and elastic recovery for data-parallel jobs (the reference defines
`Heartbeat` / `Shutdown` / `Barrier` message types but never uses them for liveness, and its accept loop
has no timeout: rust-nn src/distributed.rs:270-281, 448-457).

Every rank publishes a heartbeat counter in the TCP store. Between steps - never while a kernel or a
collective is in flight - a rank asks `ElasticGroup.dead_ranks()`; if someone has stopped beating, the
survivors call `shrink()`: they agree on the member list through the store, tear down the process group,
re-initialise it with the smaller world (ranks renumbered in order) and reload the last checkpoint. Nothing
here touches a GPU; a dead rank is noticed on the host before the next launch. Data-parallel state is
replicated (master weights after `gather_master`, optimizer moments per shard are re-initialised from the
checkpoint), so shrinking is safe for DP; tensor- / expert-parallel groups need every member and abort instead.
"""
from __future__ import annotations

import datetime
import os
import time
from typing import Callable, List, Optional

import torch.distributed as dist

from ..distributed import HeartbeatMonitor, TcpStore


class ElasticGroup:
    def __init__(self, rank: int, world_size: int, store: TcpStore, backend: str = "gloo", base_port: int = 29800,
                 heartbeat_interval: float = 0.1, heartbeat_timeout: float = 1.0, pg_timeout: float = 10.0):
        self.orig_rank, self.rank, self.world = rank, rank, world_size
        self.members: List[int] = list(range(world_size))       # original rank ids still in the job
        self.store, self.backend, self.base_port = store, backend, base_port
        self.generation = 0
        self.pg_timeout = pg_timeout
        self.monitor = HeartbeatMonitor(store, rank, world_size, heartbeat_interval, heartbeat_timeout).start()
        self._init_pg()

    def _init_pg(self) -> None:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(self.base_port + self.generation)
        dist.init_process_group(self.backend, rank=self.rank, world_size=self.world,
                                timeout=datetime.timedelta(seconds=self.pg_timeout))

    def dead_ranks(self) -> List[int]:
        """Original rank ids (among the current members) whose heartbeat has stopped."""
        return [r for r in self.monitor.dead_ranks() if r in self.members]

    def shrink(self, dead: List[int], on_reload: Optional[Callable[[], None]] = None, settle: float = 5.0) -> None:
        """Drop `dead` from the job and rebuild the process group among the survivors."""
        survivors = [r for r in self.members if r not in dead]
        if self.orig_rank not in survivors:
            raise RuntimeError("this rank was declared dead by its peers")
        gen = self.generation + 1
        # survivors agree on the member list: the lowest survivor proposes, the others confirm the same list
        key = f"__elastic__/gen{gen}/members"
        proposal = ",".join(map(str, survivors)).encode()
        if self.orig_rank == survivors[0]:
            self.store.set(key, proposal)
        agreed = self.store.get(key, wait=settle)
        if agreed is None:
            raise TimeoutError("survivors could not agree on the new member list")
        survivors = [int(x) for x in agreed.decode().split(",")]
        if not self.store.barrier(f"__elastic__/gen{gen}/ready", len(survivors), settle):
            raise TimeoutError("not every survivor reached the re-rendezvous")
        try:
            dist.destroy_process_group()
        except Exception:
            pass
        self.members, self.generation = survivors, gen
        self.rank, self.world = survivors.index(self.orig_rank), len(survivors)
        self._init_pg()
        if on_reload is not None:
            on_reload()

    def close(self) -> None:
        self.monitor.stop()
        try:
            dist.destroy_process_group()
        except Exception:
            pass
