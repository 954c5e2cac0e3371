"""Point-to-point byte and tensor transport over TCP sockets between the nodes of an expert-parallel cluster: the portable
form of the reference's ``TCPCommBackend`` (include/oil/expert_parallel.h:91-115; its implementation is Winsock,
src/expert_parallel.cpp:69-272).

Inside one machine the framework moves tokens over NVLink peer memory and bootstraps with ``torch.distributed``; this class is
the stand-alone control / fallback channel with the reference's surface: ``listen`` / ``connect`` / ``disconnect`` / ``send`` /
``recv`` / ``send_async`` / ``recv_async`` / ``wait_all`` / ``is_connected`` / ``bytes_sent`` / ``bytes_received`` /
``shutdown``. Node ids are small integers handed out per connection (the reference uses the socket handle). ``send`` writes
the bytes as they are and ``recv`` reads until ``max_bytes`` have arrived or the peer closes, as the reference does;
``send_tensor`` / ``recv_tensor`` add a header (dtype, shape) so that the receiver needs no side knowledge. The asynchronous
forms really are asynchronous here (one worker thread per connection and direction); ``wait_all`` joins them.
"""
from __future__ import annotations

import socket
import struct
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.uint8, torch.int8, torch.float64, torch.bool]


class _Conn:
    def __init__(self, sock: socket.socket, address: str, port: int):
        self.sock, self.address, self.port = sock, address, port
        self.connected = True
        self.bytes_sent = self.bytes_received = 0
        self.send_lock, self.recv_lock = threading.Lock(), threading.Lock()
        self.tx = ThreadPoolExecutor(max_workers=1)
        self.rx = ThreadPoolExecutor(max_workers=1)


class TCPCommBackend:
    CHUNK = 65536

    def __init__(self):
        self._lock = threading.Lock()
        self._conns: Dict[int, _Conn] = {}
        self._next_id = 0
        self._listener: Optional[socket.socket] = None
        self._accept_thread: Optional[threading.Thread] = None
        self._running = False
        self._pending: List[Future] = []
        self.port = 0

    # ---- connections
    def listen(self, port: int, host: str = "0.0.0.0") -> bool:
        try:
            s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            s.bind((host, port))
            s.listen(64)
        except (OSError, OverflowError):       # port in use, out of range, ...
            return False
        self._listener, self.port, self._running = s, s.getsockname()[1], True
        self._accept_thread = threading.Thread(target=self._accept_loop, daemon=True)
        self._accept_thread.start()
        return True

    def _accept_loop(self):
        while self._running:
            try:
                c, (addr, port) = self._listener.accept()
            except OSError:
                return
            self._add(c, addr, port)

    def _add(self, sock: socket.socket, address: str, port: int) -> int:
        sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        with self._lock:
            nid = self._next_id
            self._next_id += 1
            self._conns[nid] = _Conn(sock, address, port)
        return nid

    def connect(self, address: str, port: int, timeout: float = 10.0) -> int:
        """-> node id of the new connection, or -1 (the reference returns a bool and uses the socket handle as the id)."""
        try:
            s = socket.create_connection((address, port), timeout=timeout)
            s.settimeout(None)
        except (OSError, OverflowError):
            return -1
        return self._add(s, address, port)

    def nodes(self) -> List[int]:
        with self._lock:
            return sorted(self._conns)

    def disconnect(self, node_id: int):
        with self._lock:
            c = self._conns.pop(node_id, None)
        if c is not None:
            c.connected = False
            try:
                c.sock.shutdown(socket.SHUT_RDWR)
            except OSError:
                pass
            c.sock.close()
            c.tx.shutdown(wait=False)
            c.rx.shutdown(wait=False)

    def is_connected(self, node_id: int) -> bool:
        with self._lock:
            c = self._conns.get(node_id)
        return c is not None and c.connected

    def _get(self, node_id: int) -> Optional[_Conn]:
        with self._lock:
            c = self._conns.get(node_id)
        return c if c is not None and c.connected else None

    # ---- bytes
    def send(self, node_id: int, data) -> bool:
        c = self._get(node_id)
        if c is None:
            return False
        view = memoryview(data).cast("B")
        with c.send_lock:
            try:
                for lo in range(0, len(view), self.CHUNK):
                    c.sock.sendall(view[lo:lo + self.CHUNK])
            except OSError:
                c.connected = False
                return False
            c.bytes_sent += len(view)
        return True

    def recv(self, node_id: int, max_bytes: int) -> Optional[bytes]:
        """Up to ``max_bytes``: returns once they have all arrived or the peer has closed; None when nothing arrived."""
        c = self._get(node_id)
        if c is None:
            return None
        buf = bytearray()
        with c.recv_lock:
            while len(buf) < max_bytes:
                try:
                    got = c.sock.recv(min(self.CHUNK, max_bytes - len(buf)))
                except OSError:
                    got = b""
                if not got:
                    c.connected = False
                    break
                buf += got
            c.bytes_received += len(buf)
        return bytes(buf) if buf else None

    def send_async(self, node_id: int, data) -> Future:
        c = self._get(node_id)
        if c is None:
            f: Future = Future()
            f.set_result(False)
            return f
        f = c.tx.submit(self.send, node_id, bytes(memoryview(data).cast("B")))     # the caller may reuse its buffer at once
        with self._lock:
            self._pending.append(f)
        return f

    def recv_async(self, node_id: int, max_bytes: int) -> Future:
        c = self._get(node_id)
        if c is None:
            f: Future = Future()
            f.set_result(None)
            return f
        f = c.rx.submit(self.recv, node_id, max_bytes)
        with self._lock:
            self._pending.append(f)
        return f

    def wait_all(self):
        with self._lock:
            pending, self._pending = self._pending, []
        for f in pending:
            f.result()

    # ---- tensors: header = magic, dtype code, rank, dims..., then the raw little-endian payload
    def send_tensor(self, node_id: int, t: torch.Tensor) -> bool:
        t = t.detach().cpu().contiguous()
        hdr = struct.pack("<IBB", 0x4F494C54, _DTYPES.index(t.dtype), t.dim()) + struct.pack(f"<{t.dim()}q", *t.shape)
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        return self.send(node_id, hdr + raw)

    def recv_tensor(self, node_id: int) -> Optional[torch.Tensor]:
        head = self.recv(node_id, 6)
        if head is None or len(head) < 6:
            return None
        magic, code, rank = struct.unpack("<IBB", head)
        if magic != 0x4F494C54 or code >= len(_DTYPES) or rank > 8:
            raise ValueError("recv_tensor: not a tensor frame")
        dims: Tuple[int, ...] = ()
        if rank:
            d = self.recv(node_id, 8 * rank)
            if d is None or len(d) < 8 * rank:
                return None
            dims = struct.unpack(f"<{rank}q", d)
        dtype = _DTYPES[code]
        n = int(np.prod(dims)) if dims else 1
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        raw = self.recv(node_id, nbytes) if nbytes else b""
        if raw is None or len(raw) < nbytes:
            return None
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dtype).reshape(dims) if nbytes else torch.empty(dims, dtype=dtype)

    # ---- statistics and teardown
    def bytes_sent(self, node_id: int) -> int:
        c = self._conns.get(node_id)
        return c.bytes_sent if c else 0

    def bytes_received(self, node_id: int) -> int:
        c = self._conns.get(node_id)
        return c.bytes_received if c else 0

    def shutdown(self):
        self._running = False
        if self._listener is not None:
            try:
                self._listener.close()
            except OSError:
                pass
            self._listener = None
        for nid in self.nodes():
            self.disconnect(nid)
