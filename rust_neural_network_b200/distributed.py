"""Distributed-training API of the reference (rust-nn src/distributed.rs) plus the host-side runtime
around the real multi-GPU paths.

Reference surface kept: `DistributedConfig` (`effective_lr`, `shard_range`, `local_batch_size`),
`ring_all_reduce_simulated` / `ring_all_reduce_all` / `average_gradients` (the CPU restatement that
serves as the ORACLE of the fused reduce-scatter kernel), `flatten_gradients` / `unflatten_gradients` /
`sync_gradients` / `clip_gradients`, `Message` / `MessageType` with the byte-exact
`[type u8][len u32 LE][payload]` framing, `send_message` / `recv_message`, and `DistributedWorker`
(`standalone`, `connect`, `train_step`).

Added (the reference has none of it): a TCP key-value store in C++ (`TcpStore`) for rendezvous,
`HeartbeatMonitor` for host-side failure detection, and `init_from_env()` which honours the
reference's documented-but-unused `RUST_NN_RANK / RUST_NN_WORLD_SIZE / RUST_NN_MASTER` variables as
aliases of `RANK / WORLD_SIZE / MASTER_ADDR:MASTER_PORT`. Gradients of real multi-GPU jobs move
through `parallel.ddp.DistributedAdam`, never through these sockets.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import enum
import os
import socket
import struct
import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _native as nv

_P = C.c_void_p
nv.register_sigs({
    "b200_msg_serialize": [C.c_int, _P, C.c_longlong, _P, C.c_longlong],
    "b200_msg_deserialize": [_P, C.c_longlong, C.POINTER(C.c_int)],
    "b200_store_server_start": [C.c_int, C.POINTER(C.c_int)],
    "b200_store_server_stop": [_P],
    "b200_store_connect": [C.c_char_p, C.c_int, C.c_int],
    "b200_store_close": [C.c_longlong],
    "b200_store_set": [C.c_longlong, C.c_char_p, _P, C.c_longlong, C.c_int],
    "b200_store_get": [C.c_longlong, C.c_char_p, _P, C.c_longlong, C.c_int],
    "b200_store_add": [C.c_longlong, C.c_char_p, C.c_longlong, C.c_int],
})


def _host():
    lib = nv.host()
    lib.b200_msg_serialize.restype = C.c_longlong
    lib.b200_msg_deserialize.restype = C.c_longlong
    lib.b200_store_server_start.restype = C.c_void_p
    lib.b200_store_server_stop.restype = None
    lib.b200_store_connect.restype = C.c_longlong
    lib.b200_store_close.restype = None
    lib.b200_store_get.restype = C.c_longlong
    lib.b200_store_add.restype = C.c_longlong
    return lib


# ----------------------------------------------------------------------------- all-reduce oracle
def ring_all_reduce_simulated(local_data: List[float], all_workers: List[List[float]], rank: int, world_size: int) -> None:
    """In-place ring all-reduce of `local_data` against the other workers' buffers, chunk = ceil(n/world),
    2(N-1) rounds (src/distributed.rs:54-102). Lists (or 1-D tensors) are updated in place."""
    if world_size <= 1:
        return
    n = len(local_data)
    chunk = -(-n // world_size)
    left = (rank + world_size - 1) % world_size
    for rnd in range(world_size - 1):
        ridx = (rank - rnd - 1 + world_size) % world_size
        a, b = ridx * chunk, min(ridx * chunk + chunk, n)
        for i in range(a, b):
            local_data[i] += all_workers[left][i]
        all_workers[rank][a:b] = local_data[a:b]
    for rnd in range(world_size - 1):
        ridx = (rank - rnd + world_size) % world_size
        a, b = ridx * chunk, min(ridx * chunk + chunk, n)
        local_data[a:b] = all_workers[left][a:b]
        all_workers[rank][a:b] = local_data[a:b]


def ring_all_reduce_all(workers: List, world_size: int) -> None:
    """Element-wise sum over all workers written back to every worker (src/distributed.rs:107-124)."""
    if world_size <= 1:
        return
    if isinstance(workers[0], torch.Tensor):
        s = torch.stack(list(workers)).sum(0)
        for w in workers:
            w.copy_(s)
        return
    n = len(workers[0])
    s = [sum(w[i] for w in workers) for i in range(n)]
    for w in workers:
        w[:] = s


def average_gradients(data, world_size: int) -> None:
    if isinstance(data, torch.Tensor):
        data.mul_(1.0 / world_size)
    else:
        for i in range(len(data)):
            data[i] *= 1.0 / world_size


def flatten_gradients(params) -> torch.Tensor:
    """One flat fp32 bucket of all gradients (zeros where a parameter has none), src/distributed.rs:140-151."""
    parts = [(p.grad if p.grad is not None else torch.zeros_like(p)).detach().float().reshape(-1) for p in params]
    return torch.cat(parts) if parts else torch.zeros(0)


def unflatten_gradients(params, flat: torch.Tensor) -> None:
    off = 0
    for p in params:
        n = p.numel()
        g = flat[off:off + n].view(p.shape).to(p.device, p.dtype)
        if p.grad is None:
            p.grad = g.clone()
        else:
            p.grad.copy_(g)
        off += n


def sync_gradients(params, world_size: int, other_worker_grads: Sequence, rank: int) -> None:
    """Average the local gradients with the other workers' flat gradient buffers (src/distributed.rs:170-196)."""
    if world_size <= 1:
        return
    local = flatten_gradients(params)
    workers, it = [], iter(other_worker_grads)
    for r in range(world_size):
        if r == rank:
            workers.append(local)
        else:
            workers.append(torch.as_tensor(next(it), dtype=torch.float32).to(local.device).reshape(-1))
    ring_all_reduce_all(workers, world_size)
    average_gradients(local, world_size)
    unflatten_gradients(params, local)


def clip_gradients(params, max_norm: float) -> float:
    """Scale all gradients so that their global L2 norm is at most `max_norm` (src/distributed.rs:507-523)."""
    total = 0.0
    for p in params:
        if p.grad is not None:
            total += float((p.grad.float() ** 2).sum())
    total = total ** 0.5
    if total > max_norm:
        s = max_norm / total
        for p in params:
            if p.grad is not None:
                p.grad.mul_(s)
    return total


# ----------------------------------------------------------------------------- config
@dataclasses.dataclass
class DistributedConfig:
    rank: int = 0
    world_size: int = 1
    scale_lr: bool = True
    grad_clip: float = 0.0

    @staticmethod
    def single() -> "DistributedConfig":
        return DistributedConfig()

    @staticmethod
    def new(rank: int, world_size: int) -> "DistributedConfig":
        return DistributedConfig(rank, world_size)

    def effective_lr(self, base_lr: float) -> float:
        return base_lr * self.world_size if self.scale_lr else base_lr

    def shard_range(self, total_samples: int) -> Tuple[int, int]:
        per, rem = divmod(total_samples, self.world_size)
        start = self.rank * per + min(self.rank, rem)
        end = start + per + (1 if self.rank < rem else 0)
        return start, min(end, total_samples)

    def local_batch_size(self, global_batch_size: int) -> int:
        return max(global_batch_size // self.world_size, 1)


def init_from_env() -> DistributedConfig:
    """Rank / world size from RANK / WORLD_SIZE, falling back to the reference's RUST_NN_* names."""
    rank = int(os.environ.get("RANK", os.environ.get("RUST_NN_RANK", "0")))
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("RUST_NN_WORLD_SIZE", "1")))
    master = os.environ.get("RUST_NN_MASTER")
    if master and "MASTER_ADDR" not in os.environ:
        host, _, port = master.partition(":")
        os.environ["MASTER_ADDR"] = host or "127.0.0.1"
        if port:
            os.environ.setdefault("MASTER_PORT", port)
    return DistributedConfig(rank, world)


# ----------------------------------------------------------------------------- messages
class MessageType(enum.IntEnum):
    GradientChunk = 0
    Barrier = 1
    Heartbeat = 2
    Shutdown = 3
    Parameters = 4


@dataclasses.dataclass
class Message:
    msg_type: MessageType
    payload: bytes = b""

    @staticmethod
    def gradient_chunk(data) -> "Message":
        arr = np.asarray(data, dtype="<f4")
        return Message(MessageType.GradientChunk, arr.tobytes())

    @staticmethod
    def barrier() -> "Message":
        return Message(MessageType.Barrier, b"")

    @staticmethod
    def heartbeat(rank: int = 0) -> "Message":
        return Message(MessageType.Heartbeat, struct.pack("<I", rank))

    def serialize(self) -> bytes:
        lib = _host()
        out = np.empty(5 + len(self.payload), dtype=np.uint8)
        pl = np.frombuffer(self.payload, dtype=np.uint8) if self.payload else np.empty(0, dtype=np.uint8)
        n = lib.b200_msg_serialize(int(self.msg_type), pl.ctypes.data if len(pl) else None, len(pl), out.ctypes.data, out.size)
        if n < 0:
            raise ValueError("message too large")
        return out[:n].tobytes()

    @staticmethod
    def deserialize(data: bytes) -> Optional["Message"]:
        """None for truncated frames and unknown types (src/distributed.rs:308-333)."""
        lib = _host()
        arr = np.frombuffer(data, dtype=np.uint8)
        t = C.c_int(0)
        n = lib.b200_msg_deserialize(arr.ctypes.data if arr.size else None, arr.size, C.byref(t))
        if n < 0:
            return None
        return Message(MessageType(t.value), bytes(data[5:5 + n]))

    def as_floats(self) -> List[float]:
        n = len(self.payload) // 4
        return np.frombuffer(self.payload[: 4 * n], dtype="<f4").tolist()


def send_message(sock: socket.socket, msg: Message) -> None:
    sock.sendall(msg.serialize())


def recv_message(sock: socket.socket, timeout: Optional[float] = 30.0) -> Message:
    sock.settimeout(timeout)

    def read(n):
        buf = b""
        while len(buf) < n:
            part = sock.recv(n - len(buf))
            if not part:
                raise ConnectionError("peer closed the connection")
            buf += part
        return buf
    hdr = read(5)
    (ln,) = struct.unpack("<I", hdr[1:5])
    msg = Message.deserialize(hdr + read(ln))
    if msg is None:
        raise ValueError("Failed to deserialize message")
    return msg


# ----------------------------------------------------------------------------- TCP store + liveness
class TcpStore:
    """Key-value store over the framing above (C++ server thread + blocking client with deadlines)."""

    def __init__(self, host: str = "127.0.0.1", port: int = 0, is_master: bool = False, timeout: float = 30.0):
        lib = _host()
        self._lib, self._server, self.host = lib, None, host
        if is_master:
            bound = C.c_int(0)
            self._server = lib.b200_store_server_start(port, C.byref(bound))
            if not self._server:
                raise OSError(f"cannot bind store server on port {port}")
            port = bound.value
        self.port = port
        self._fd = lib.b200_store_connect(host.encode(), port, int(timeout * 1000))
        if self._fd < 0:
            raise ConnectionError(f"cannot reach store at {host}:{port}")
        self._lock = threading.Lock()

    def set(self, key: str, value: bytes, timeout: float = 10.0) -> None:
        arr = np.frombuffer(value, dtype=np.uint8) if value else np.empty(0, dtype=np.uint8)
        with self._lock:
            rc = self._lib.b200_store_set(self._fd, key.encode(), arr.ctypes.data if arr.size else None, arr.size, int(timeout * 1000))
        if rc != 0:
            raise ConnectionError("store set failed")

    def get(self, key: str, wait: float = 10.0) -> Optional[bytes]:
        """Value of `key`, waiting up to `wait` seconds for it to appear; None on expiry."""
        out = np.empty(1 << 20, dtype=np.uint8)
        with self._lock:
            n = self._lib.b200_store_get(self._fd, key.encode(), out.ctypes.data, out.size, int(wait * 1000))
        if n == -2:
            return None
        if n < 0:
            raise ConnectionError("store get failed")
        return out[:n].tobytes()

    def add(self, key: str, delta: int, timeout: float = 10.0) -> int:
        with self._lock:
            v = self._lib.b200_store_add(self._fd, key.encode(), delta, int(timeout * 1000))
        if v == -(1 << 63):
            raise ConnectionError("store add failed")
        return v

    def barrier(self, name: str, world_size: int, timeout: float = 30.0) -> bool:
        """True if all `world_size` ranks arrived within `timeout` seconds."""
        n = self.add(f"__barrier__/{name}", 1)
        if n >= world_size:
            self.set(f"__barrier__/{name}/done", b"1")
            return True
        return self.get(f"__barrier__/{name}/done", wait=timeout) is not None

    def close(self):
        if self._fd >= 0:
            self._lib.b200_store_close(self._fd); self._fd = -1
        if self._server:
            self._lib.b200_store_server_stop(self._server); self._server = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HeartbeatMonitor:
    """Host-side failure detection: every rank publishes a heartbeat counter to the store; `dead_ranks()`
    lists ranks whose counter has not advanced for `timeout` seconds. Nothing here touches a GPU: a
    rank that died is noticed on the host, before the survivors launch their next step."""

    def __init__(self, store: TcpStore, rank: int, world_size: int, interval: float = 0.2, timeout: float = 2.0):
        self.store, self.rank, self.world, self.interval, self.timeout = store, rank, world_size, interval, timeout
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._last: Dict[int, Tuple[int, float]] = {}

    def start(self):
        def beat():
            while not self._stop.is_set():
                try:
                    self.store.add(f"__hb__/{self.rank}", 1)
                except Exception:
                    return
                self._stop.wait(self.interval)
        self._thread = threading.Thread(target=beat, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def dead_ranks(self) -> List[int]:
        now, dead = time.time(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self.store.add(f"__hb__/{r}", 0)
            prev = self._last.get(r)
            if prev is None or v != prev[0]:
                self._last[r] = (v, now)
            elif now - prev[1] > self.timeout:
                dead.append(r)
        return dead


# ----------------------------------------------------------------------------- worker
class DistributedWorker:
    """`standalone(rank, world)` needs no network; `connect(...)` performs a rendezvous through a
    `TcpStore` (with a deadline) instead of the reference's unbounded accept loop. `train_step`
    follows src/distributed.rs:472-503: local forward/backward, gradient averaging with the other
    workers' flat gradients, optional clipping, optimizer step; returns loss / batch rows."""

    def __init__(self, config: DistributedConfig, store: Optional[TcpStore] = None):
        self.config, self.store = config, store

    @staticmethod
    def standalone(rank: int, world_size: int) -> "DistributedWorker":
        return DistributedWorker(DistributedConfig(rank, world_size))

    @staticmethod
    def connect(rank: int, world_size: int, master_host: str = "127.0.0.1", master_port: int = 29400, timeout: float = 30.0) -> "DistributedWorker":
        store = TcpStore(master_host, master_port, is_master=(rank == 0), timeout=timeout)
        store.set(f"rank/{rank}", Message.heartbeat(rank).serialize())
        if not store.barrier("connect", world_size, timeout):
            store.close()
            raise TimeoutError(f"rendezvous of {world_size} ranks did not complete within {timeout}s")
        return DistributedWorker(DistributedConfig(rank, world_size), store)

    def train_step(self, model, optimizer, loss_fn, inputs, targets, other_worker_grads: Sequence = ()) -> float:
        optimizer.zero_grad()
        loss = loss_fn(model(inputs), targets)
        loss.backward()
        params = model.parameters()
        sync_gradients(params, self.config.world_size, other_worker_grads, self.config.rank)
        if self.config.grad_clip > 0:
            clip_gradients(params, self.config.grad_clip)
        optimizer.step()
        return float(loss.detach()) / max(inputs.shape[0], 1)


from ._compat import alias_fields as _alias_fields  # noqa: E402

# src/distributed.rs:382-388: the ring's sockets. Here the ring runs over the C++ TCP store, so the "connections" are the
# store handle (None until `connect`) in both directions.
_alias_fields(DistributedWorker, right_conn=lambda self: self.store, left_conn=lambda self: self.store)
