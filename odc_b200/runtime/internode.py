"""Inter-node data path: one-sided ``get`` / ``add`` on a remote rank's heap region, served over TCP.

Ranks of other nodes are not mapped into this rank's address space, so a shard there is named by
its heap OFFSET (the allocator is deterministic, offsets are equal on every rank) and moved by a
small server that every rank runs next to its trainer:

* ``GET  offset, numel, dtype``  ->  the bytes of that range of the server's own region;
* ``ADD  offset, numel, src dtype, dst dtype, scale, counter offset`` + payload  ->  the server adds
  ``scale * payload`` into its region (atomically with respect to same-node producers: the GPU path
  uses the same ``red.add`` kernel as NVLink peers, the CPU path takes the owner's file lock) and
  then counts one arrival on the counter, exactly what a same-node producer does.  A contribution
  larger than the staging cap travels as several ``ADD`` messages on one connection; all but the
  last carry counter offset -1 and count nothing, and the server handles a connection's messages
  in order, so the arrival still means "the whole contribution has been added".

The trainer of the serving rank never takes part (the server threads do), so the on-demand
property holds across nodes: a rank can pull parameters from, and push gradients to, a rank that is
busy with a different number of microbatches.  On GPUs the payload is staged through pinned host
memory on both sides; this is the portable path of this build (the image has neither an RDMA verbs
library nor NVSHMEM), and the wire format is the only thing an RDMA transport would replace.

Exposure.  The server reads and writes training state, so it is closed by default: the listener binds
to the loopback address only, which serves every job whose ranks share one host (emulated nodes).  A
job that really spans hosts must name, per rank, the one interface address to bind and advertise in
``ODC_HOST_ADDR`` (never the wildcard address).  In both cases a connection is served only after it
has answered a challenge with an HMAC of a per-job secret that rank 0 draws at start-up and shares
over the control group, so another process that can reach the port cannot read or modify the heap.

Role in the reference: the NVSHMEM get/put kernels for peers on other nodes and the request/ack
words served by the watcher process (odc/primitives/gather.py:22-64,129-175,
odc/primitives/scatter_accumulate.py:42-174,291-401).
"""
from __future__ import annotations

import hashlib
import hmac
import logging
import os
import socket
import struct
import threading
from typing import Dict, List, Sequence, Tuple

import torch

from .. import config
from . import control
from .heap import SymmetricHeap
from .status import OdcTimeoutError

logger = logging.getLogger("odc_b200")

_DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32, torch.int16,
           torch.int8, torch.uint8, torch.bool]
_CODE = {dt: i for i, dt in enumerate(_DTYPES)}
_MAGIC = b"ODC1"
# magic, op, src dtype, dst dtype, pad, offset, numel, counter offset, scale
_HDR = struct.Struct("<4sBBBxqqqd")
_REPLY = struct.Struct("<Bxxxq")  # status (0 = ok), payload bytes that follow (data or an error message)
OP_GET, OP_ADD, OP_BYE = 1, 2, 3


def _itemsize(dt: torch.dtype) -> int:
    return torch.empty((), dtype=dt).element_size()


def _recv_exact(sock: socket.socket, view: memoryview) -> None:
    got = 0
    n = len(view)
    while got < n:
        try:
            k = sock.recv_into(view[got:], n - got)
        except socket.timeout as e:
            raise OdcTimeoutError(f"inter-node transfer stalled after {got} of {n} bytes") from e
        if k == 0:
            raise ConnectionError("peer closed the connection in the middle of a message")
        got += k


def _host_buffer(nbytes: int, pinned: bool) -> torch.Tensor:
    t = torch.empty(max(nbytes, 1), dtype=torch.uint8)
    return t.pin_memory() if pinned else t


def _bind_address() -> str:
    """Loopback unless the user names this rank's interface address in ``ODC_HOST_ADDR``."""
    addr = os.environ.get("ODC_HOST_ADDR", "127.0.0.1").strip()
    if addr in ("", "0.0.0.0", "::", "*"):
        raise ValueError("ODC_HOST_ADDR must name one interface address; the wildcard address is not accepted")
    return addr


class InterNodeEndpoint:
    """Server threads for this rank's region plus one client connection per rank of other nodes."""

    def __init__(self, heap: SymmetricHeap):
        self.heap = heap
        self.rank = heap.rank
        self.cuda = heap.device.type == "cuda"
        self.timeout_s = config.wait_timeout_ms() / 1e3
        self._closing = False
        self._listener = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._listener.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        addr = _bind_address()
        self._listener.bind((addr, 0))
        self._listener.listen(128)
        port = self._listener.getsockname()[1]
        # per-job secret: only holders may use the server (challenge / response on every new connection)
        self._secret: bytes = control.broadcast_object(os.urandom(32) if self.rank == 0 else None, src=0)
        info = control.all_gather_object((addr, port, socket.gethostname()))
        self.addresses: List[Tuple[str, int]] = [(a, p) for a, p, _ in info]
        hosts = {h for _, _, h in info}
        if len(hosts) > 1 and any(a.startswith("127.") for a, _, _ in info):
            self._listener.close()
            raise RuntimeError("the job spans several hosts but some ranks listen on loopback only: set "
                               "ODC_HOST_ADDR on every rank to the address its peers should connect to")
        self._conns: Dict[int, socket.socket] = {}
        self._conn_locks: Dict[int, threading.Lock] = {}
        self._handlers: List[threading.Thread] = []
        self._tables: Dict[int, torch.Tensor] = {}
        self.served = {"get": 0, "add": 0}
        self.rejected = 0  # connections that failed the challenge
        self._stat_lock = threading.Lock()  # the counters are bumped from several server threads
        self.sent = {"get": 0, "add": 0, "bytes": 0}
        if self.cuda:
            from .. import _ext
            self._ext = _ext.load()
            self._stream = torch.cuda.Stream(device=heap.device)
            self._status = torch.zeros(4, dtype=torch.int32, device=heap.device)
            self._status_hosts: Dict[int, torch.Tensor] = {}
            # arrivals of all but the last piece of a split contribution are counted here and ignored
            self._scratch_counter = torch.zeros(8, dtype=torch.int64, device=heap.device)
            self._scratch_counter_table = torch.tensor([self._scratch_counter.data_ptr()], dtype=torch.int64,
                                                       device=heap.device)
            torch.cuda.current_stream().synchronize()
        self._acceptor = threading.Thread(target=self._accept_loop, name="odc-internode-accept", daemon=True)
        self._acceptor.start()
        control.host_barrier()  # every listener is up before anyone connects

    # ------------------------------------------------------------------------------- server
    def _accept_loop(self) -> None:
        while not self._closing:
            try:
                conn, _ = self._listener.accept()
            except OSError:
                return
            conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            t = threading.Thread(target=self._serve, args=(conn,), name="odc-internode-serve", daemon=True)
            t.start()
            self._handlers = [h for h in self._handlers if h.is_alive()] + [t]

    def _authenticate(self, conn: socket.socket) -> bool:
        nonce = os.urandom(16)
        answer = bytearray(32)
        try:
            conn.settimeout(10.0)
            conn.sendall(nonce)
            _recv_exact(conn, memoryview(answer))
            conn.settimeout(None)
        except (OSError, ConnectionError, OdcTimeoutError):
            return False
        return hmac.compare_digest(bytes(answer), hmac.new(self._secret, nonce, hashlib.sha256).digest())

    def _serve(self, conn: socket.socket) -> None:
        if not self._authenticate(conn):
            with self._stat_lock:
                self.rejected += 1
            conn.close()
            return
        if self.cuda:
            torch.cuda.set_device(self.heap.device)
        hdr = bytearray(_HDR.size)
        staging = _host_buffer(1 << 20, self.cuda)
        try:
            while True:
                try:
                    _recv_exact(conn, memoryview(hdr))
                except (ConnectionError, OSError):
                    return
                magic, op, src_c, dst_c, offset, numel, ctr_off, scale = _HDR.unpack(hdr)
                if magic != _MAGIC or op == OP_BYE:
                    return
                if (numel < 0 or offset < 0 or src_c >= len(_DTYPES) or dst_c >= len(_DTYPES)
                        or numel * 8 > getattr(self.heap, "nbytes", 1 << 62) * 8):
                    return  # malformed header: the byte stream cannot be trusted any further
                try:
                    if op == OP_GET:
                        dt = _DTYPES[src_c]
                        nb = numel * _itemsize(dt)
                        if staging.numel() < nb:
                            staging = _host_buffer(nb, self.cuda)
                        self._read_region(offset, numel, dt, staging)
                        conn.sendall(_REPLY.pack(0, nb))
                        conn.sendall(memoryview(staging.numpy())[:nb])
                        with self._stat_lock:
                            self.served["get"] += 1
                    elif op == OP_ADD:
                        src_dt, dst_dt = _DTYPES[src_c], _DTYPES[dst_c]
                        nb = numel * _itemsize(src_dt)
                        if staging.numel() < nb:
                            staging = _host_buffer(nb, self.cuda)
                        _recv_exact(conn, memoryview(staging.numpy())[:nb])
                        self._add_region(offset, numel, src_dt, dst_dt, scale, ctr_off, staging)
                        conn.sendall(_REPLY.pack(0, 0))
                        with self._stat_lock:
                            self.served["add"] += 1
                    else:
                        raise ValueError(f"unknown operation {op}")
                except (IndexError, ValueError, RuntimeError) as e:  # report to the client, keep serving
                    msg = f"rank {self.rank}: {type(e).__name__}: {e}".encode()
                    conn.sendall(_REPLY.pack(1, len(msg)) + msg)
        finally:
            conn.close()

    def _read_region(self, offset: int, numel: int, dt: torch.dtype, staging: torch.Tensor) -> None:
        src = self.heap.local(offset, numel, dt)  # raises IndexError outside the region
        dst = staging[: numel * _itemsize(dt)].view(dt)
        if self.cuda:
            with torch.cuda.stream(self._stream):
                dst.copy_(src, non_blocking=True)
            self._stream.synchronize()
        else:
            dst.copy_(src)

    def _add_region(self, offset: int, numel: int, src_dt: torch.dtype, dst_dt: torch.dtype, scale: float,
                    ctr_off: int, staging: torch.Tensor) -> None:
        acc = self.heap.local(offset, numel, dst_dt)
        ctr = self.heap.local(ctr_off, 1, torch.int64) if ctr_off >= 0 else None
        payload = staging[: numel * _itemsize(src_dt)].view(src_dt)
        if self.cuda:
            with torch.cuda.stream(self._stream):
                dev = payload.to(self.heap.device, non_blocking=True)
                # same kernel as a same-node producer, with this rank as the only owner: vector red.add into
                # the accumulator, then a release-ordered arrival on the counter
                ctr_table = self._table(ctr_off) if ctr_off >= 0 else self._scratch_counter_table
                self._ext.scatter_accumulate(dev.view(1, numel), self._table(offset), ctr_table, numel,
                                             dst_dt, 0, float(scale), config.debug_bounds(), self._status)
                # the status word is read on this stream too: a copy on the default stream would queue behind
                # whatever the trainer has running there
                host_status = self._status_host(threading.get_ident())
                host_status.copy_(self._status, non_blocking=True)
            self._stream.synchronize()
            code = int(host_status[0])
            if code != 0:
                with torch.cuda.stream(self._stream):
                    self._status.zero_()
                self._stream.synchronize()
                raise RuntimeError(f"accumulation kernel reported error {code}")
        else:
            with self.heap.owner_lock(self.rank):
                acc.add_(payload.to(dst_dt), alpha=scale) if scale != 1.0 else acc.add_(payload.to(dst_dt))
                if ctr is not None:
                    ctr[0] += 1

    def _status_host(self, tid: int) -> torch.Tensor:
        t = self._status_hosts.get(tid)
        if t is None:
            t = self._status_hosts[tid] = torch.zeros(4, dtype=torch.int32).pin_memory()
        return t

    def _table(self, offset: int) -> torch.Tensor:
        t = self._tables.get(offset)
        if t is None:
            t = torch.tensor([self.heap.peer_ptr(self.rank, offset)], dtype=torch.int64).pin_memory().to(
                self.heap.device, non_blocking=True)  # issued on the caller's (server) stream
            self._tables[offset] = t
        return t

    # ------------------------------------------------------------------------------- client
    def _conn(self, r: int) -> socket.socket:
        c = self._conns.get(r)
        if c is None:
            c = socket.create_connection(self.addresses[r], timeout=self.timeout_s)
            c.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            c.settimeout(self.timeout_s)
            nonce = bytearray(16)
            _recv_exact(c, memoryview(nonce))
            c.sendall(hmac.new(self._secret, bytes(nonce), hashlib.sha256).digest())
            self._conns[r] = c
        return c

    def _lock(self, r: int) -> threading.Lock:
        return self._conn_locks.setdefault(r, threading.Lock())

    def _read_reply(self, r: int, into: memoryview = None) -> None:
        c = self._conns[r]
        head = bytearray(_REPLY.size)
        _recv_exact(c, memoryview(head))
        status, nb = _REPLY.unpack(head)
        if status != 0:
            msg = bytearray(nb)
            _recv_exact(c, memoryview(msg))
            raise RuntimeError(f"remote operation on rank {r} failed: {msg.decode(errors='replace')}")
        if nb:
            if into is None or len(into) != nb:
                raise RuntimeError(f"rank {r} answered with {nb} bytes, expected {0 if into is None else len(into)}")
            _recv_exact(c, into)

    def get_many(self, ranks: Sequence[int], offset: int, numel: int, dt: torch.dtype) -> List[torch.Tensor]:
        """Fetch ``[offset, offset + numel)`` of every rank in ``ranks``; returns host tensors (pinned on GPU jobs)."""
        ranks = list(ranks)
        nb = numel * _itemsize(dt)
        bufs = [_host_buffer(nb, self.cuda) for _ in ranks]
        order = sorted(range(len(ranks)), key=lambda i: ranks[i])  # one global lock order
        for i in order:
            self._lock(ranks[i]).acquire()
        try:
            # all requests go out before the first answer is read, so the owners work concurrently
            for i in order:
                self._conn(ranks[i]).sendall(_HDR.pack(_MAGIC, OP_GET, _CODE[dt], _CODE[dt], offset, numel, 0, 1.0))
            for i in order:
                self._read_reply(ranks[i], memoryview(bufs[i].numpy())[:nb])
        except (OSError, ConnectionError, OdcTimeoutError, RuntimeError):
            self._drop(ranks)  # answers of the other owners may still be queued on their connections
            raise
        finally:
            for i in order:
                self._lock(ranks[i]).release()
        self.sent["get"] += len(ranks)
        self.sent["bytes"] += nb * len(ranks)
        return [b[:nb].view(dt) for b in bufs]

    def add_many(self, ranks: Sequence[int], rows: Sequence[torch.Tensor], offset: int, dst_dt: torch.dtype,
                 ctr_offset: int, scale: float) -> None:
        """``region[offset:] of ranks[i] += scale * rows[i]`` (host tensors), then one arrival on each counter.

        ``ctr_offset = -1``: no arrival is counted (a piece of a contribution that is not its last).
        """
        ranks = list(ranks)
        order = sorted(range(len(ranks)), key=lambda i: ranks[i])
        for i in order:
            self._lock(ranks[i]).acquire()
        try:
            for i in order:
                row = rows[i].contiguous()
                c = self._conn(ranks[i])
                c.sendall(_HDR.pack(_MAGIC, OP_ADD, _CODE[row.dtype], _CODE[dst_dt], offset, row.numel(), ctr_offset,
                                    float(scale)))
                c.sendall(memoryview(row.view(torch.uint8).numpy()))
                self.sent["bytes"] += row.numel() * row.element_size()
            for i in order:
                self._read_reply(ranks[i])
        except (OSError, ConnectionError, OdcTimeoutError, RuntimeError):
            self._drop(ranks)  # answers of the other owners may still be queued on their connections
            raise
        finally:
            for i in order:
                self._lock(ranks[i]).release()
        self.sent["add"] += len(ranks)

    def _drop(self, ranks) -> None:
        # a connection that failed in the middle of a message cannot be resynchronised
        for r in ranks:
            c = self._conns.pop(r, None)
            if c is not None:
                c.close()

    def close(self) -> None:
        """Call after a barrier: no request may be in flight.  Safe to call twice."""
        if self._closing:
            return
        self._closing = True
        for r, c in list(self._conns.items()):
            try:
                c.sendall(_HDR.pack(_MAGIC, OP_BYE, 0, 0, 0, 0, 0, 0.0))
            except OSError:
                pass
            c.close()
        self._conns.clear()
        try:
            self._listener.shutdown(socket.SHUT_RDWR)
        except OSError:
            pass
        self._listener.close()
        self._acceptor.join(timeout=2.0)
        for t in self._handlers:
            t.join(timeout=2.0)
