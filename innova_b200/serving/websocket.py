"""WebSocket endpoint for token streaming (RFC 6455 over plain sockets).

Reference behaviour covered (include/oil/production.h:183-211, ``WebSocketHandler``): an accept loop on its own port, the
opening handshake (``Sec-WebSocket-Accept`` = base64(SHA-1(key + GUID))), one thread per client, text / ping / pong /
close frames with client-to-server masking and the three payload-length encodings, ``broadcast(token)`` to every
connected client, removal of clients that closed or failed. On top of that a client may send a JSON request
``{"prompt": ..., "max_tokens": ...}``; the generate callback's pieces are streamed back to that client as text frames
followed by ``{"done": true}`` (the same callback signature as the HTTP server's).

Also the ``ErrorCode`` / ``Result`` pair of the production header (include/oil/production.h:213-232).
"""
from __future__ import annotations

import base64
import enum
import hashlib
import json
import socket
import struct
import threading
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Tuple, Union

GUID = "258EAFA5-E914-47DA-95CA-C5AB0DC85B11"
OP_CONT, OP_TEXT, OP_BINARY, OP_CLOSE, OP_PING, OP_PONG = 0x0, 0x1, 0x2, 0x8, 0x9, 0xA


class ErrorCode(enum.IntEnum):
    SUCCESS = 0
    FILE_NOT_FOUND = -1
    INVALID_FORMAT = -2
    OUT_OF_MEMORY = -3
    INVALID_ARGUMENT = -4
    IO_ERROR = -5
    NETWORK_ERROR = -6
    MODEL_ERROR = -7
    TIMEOUT = -8
    UNKNOWN = -99


@dataclass
class Result:
    code: ErrorCode = ErrorCode.SUCCESS
    message: str = ""

    def ok(self) -> bool:
        return self.code == ErrorCode.SUCCESS

    @staticmethod
    def wrap(fn: Callable, *a, **kw) -> Tuple["Result", object]:
        """Runs ``fn`` and maps the usual exceptions to codes instead of raising."""
        try:
            return Result(), fn(*a, **kw)
        except FileNotFoundError as e:
            return Result(ErrorCode.FILE_NOT_FOUND, str(e)), None
        except MemoryError as e:
            return Result(ErrorCode.OUT_OF_MEMORY, str(e)), None
        except TimeoutError as e:
            return Result(ErrorCode.TIMEOUT, str(e)), None
        except (ConnectionError, socket.error) as e:
            return Result(ErrorCode.NETWORK_ERROR, str(e)), None
        except OSError as e:
            return Result(ErrorCode.IO_ERROR, str(e)), None
        except (ValueError, TypeError, KeyError) as e:
            return Result(ErrorCode.INVALID_ARGUMENT, str(e)), None
        except Exception as e:                                   # noqa: BLE001
            return Result(ErrorCode.UNKNOWN, str(e)), None


def compute_accept_key(client_key: str) -> str:
    return base64.b64encode(hashlib.sha1((client_key.strip() + GUID).encode()).digest()).decode()


def create_frame(data: Union[str, bytes], opcode: int = OP_TEXT, mask: Optional[bytes] = None, fin: bool = True) -> bytes:
    payload = data.encode() if isinstance(data, str) else bytes(data)
    head = bytearray([(0x80 if fin else 0) | opcode])
    m = 0x80 if mask else 0
    n = len(payload)
    if n < 126:
        head.append(m | n)
    elif n < 65536:
        head.append(m | 126)
        head += struct.pack(">H", n)
    else:
        head.append(m | 127)
        head += struct.pack(">Q", n)
    if mask:
        head += mask
        payload = bytes(b ^ mask[i & 3] for i, b in enumerate(payload))
    return bytes(head) + payload


def declared_length(buf: bytes):
    """Payload length that the frame header at the start of ``buf`` announces, or None while the header is incomplete.
    Lets a receiver refuse an oversized frame before buffering it."""
    if len(buf) < 2:
        return None
    n = buf[1] & 0x7F
    if n == 126:
        return struct.unpack(">H", buf[2:4])[0] if len(buf) >= 4 else None
    if n == 127:
        return struct.unpack(">Q", buf[2:10])[0] if len(buf) >= 10 else None
    return n


def parse_frame(buf: bytes):
    """-> (payload, opcode, fin, bytes consumed) or None when ``buf`` does not hold a whole frame yet."""
    if len(buf) < 2:
        return None
    fin, opcode = bool(buf[0] & 0x80), buf[0] & 0x0F
    masked, n = bool(buf[1] & 0x80), buf[1] & 0x7F
    off = 2
    if n == 126:
        if len(buf) < 4:
            return None
        n, off = struct.unpack(">H", buf[2:4])[0], 4
    elif n == 127:
        if len(buf) < 10:
            return None
        n, off = struct.unpack(">Q", buf[2:10])[0], 10
    key = b""
    if masked:
        if len(buf) < off + 4:
            return None
        key, off = buf[off:off + 4], off + 4
    if len(buf) < off + n:
        return None
    payload = buf[off:off + n]
    if masked:
        payload = bytes(b ^ key[i & 3] for i, b in enumerate(payload))
    return payload, opcode, fin, off + n


class WebSocketHandler:
    def __init__(self, port: int = 8081, host: str = "127.0.0.1", max_message: int = 1 << 20, send_timeout: float = 30.0):
        self.port, self.host, self.max_message, self.send_timeout = port, host, max_message, send_timeout
        self.generate_cb: Optional[Callable[[str, int, bool], Union[str, Iterable[str]]]] = None
        self.on_message: Optional[Callable[[str], None]] = None
        self._sock: Optional[socket.socket] = None
        self._clients: List[socket.socket] = []
        self._send_locks = {}                 # one per client: broadcast() and a client's own stream share its socket
        self._lock = threading.Lock()
        self._threads: List[threading.Thread] = []
        self._running = False

    def set_generate_callback(self, cb):
        self.generate_cb = cb

    def is_running(self) -> bool:
        return self._running

    def client_count(self) -> int:
        with self._lock:
            return len(self._clients)

    def start(self):
        self._sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._sock.bind((self.host, self.port))
        self.port = self._sock.getsockname()[1]
        self._sock.listen(16)
        self._sock.settimeout(0.2)
        self._running = True
        t = threading.Thread(target=self._accept_loop, daemon=True)
        t.start()
        self._threads.append(t)

    def stop(self):
        self._running = False
        with self._lock:
            clients, self._clients = self._clients, []
        for c in clients:
            try:
                c.sendall(create_frame(struct.pack(">H", 1001), OP_CLOSE))
            except OSError:
                pass
            self._close(c)
        if self._sock is not None:
            self._sock.close()
            self._sock = None
        for t in self._threads:
            t.join(timeout=1.0)
        self._threads = []

    def _send(self, conn: socket.socket, frame: bytes):
        """One whole frame at a time per client, whichever thread sends it; blocking with a generous limit (the 0.2 s
        receive poll would drop a client that reads slowly)."""
        with self._lock:
            lk = self._send_locks.setdefault(conn, threading.Lock())
        with lk:
            old = conn.gettimeout()
            conn.settimeout(self.send_timeout)
            try:
                conn.sendall(frame)
            finally:
                try:
                    conn.settimeout(old)
                except OSError:
                    pass

    def broadcast(self, token: str) -> int:
        """Sends a text frame to every client; returns how many received it. Clients whose socket fails are dropped."""
        frame = create_frame(token, OP_TEXT)
        with self._lock:
            clients = list(self._clients)
        sent = 0
        for c in clients:
            try:
                self._send(c, frame)
                sent += 1
            except OSError:
                self._remove(c)
        return sent

    # -- internals ---------------------------------------------------------------------------------------------------
    def _accept_loop(self):
        while self._running:
            try:
                conn, _ = self._sock.accept()
            except socket.timeout:
                continue
            except OSError:
                break
            t = threading.Thread(target=self._client_loop, args=(conn,), daemon=True)
            t.start()
            self._threads.append(t)

    def _handshake(self, conn: socket.socket):
        """-> bytes that followed the request head (the client's first frames may share its packet), or None on failure."""
        conn.settimeout(5.0)
        data = b""
        while b"\r\n\r\n" not in data and len(data) < 16384:
            chunk = conn.recv(4096)
            if not chunk:
                return None
            data += chunk
        if b"\r\n\r\n" not in data:
            return None
        data, rest = data.split(b"\r\n\r\n", 1)
        headers = {}
        for line in data.decode("latin1").split("\r\n")[1:]:
            if ":" in line:
                k, v = line.split(":", 1)
                headers[k.strip().lower()] = v.strip()
        key = headers.get("sec-websocket-key")
        if not key or "websocket" not in headers.get("upgrade", "").lower():
            conn.sendall(b"HTTP/1.1 400 Bad Request\r\nContent-Length: 0\r\nConnection: close\r\n\r\n")
            return None
        conn.sendall(("HTTP/1.1 101 Switching Protocols\r\nUpgrade: websocket\r\nConnection: Upgrade\r\n"
                      f"Sec-WebSocket-Accept: {compute_accept_key(key)}\r\n\r\n").encode())
        return rest

    def _client_loop(self, conn: socket.socket):
        try:
            rest = self._handshake(conn)
            if rest is None:
                self._close(conn)
                return
        except OSError:
            self._close(conn)
            return
        with self._lock:
            self._clients.append(conn)
        conn.settimeout(0.2)
        buf, message = rest, b""
        try:
            while self._running:
                if not buf or parse_frame(buf) is None:
                    try:
                        chunk = conn.recv(65536)
                    except socket.timeout:
                        continue
                    if not chunk:
                        break
                    buf += chunk
                while True:
                    n = declared_length(buf)
                    if n is not None and n + len(message) > self.max_message:      # refuse before buffering the payload
                        self._send(conn, create_frame(struct.pack(">H", 1009), OP_CLOSE))
                        raise ConnectionAbortedError
                    fr = parse_frame(buf)
                    if fr is None:
                        break
                    payload, op, fin, used = fr
                    buf = buf[used:]
                    if op == OP_CLOSE:
                        self._send(conn, create_frame(payload[:2], OP_CLOSE))
                        raise ConnectionAbortedError
                    if op == OP_PING:
                        self._send(conn, create_frame(payload, OP_PONG))
                    elif op in (OP_TEXT, OP_BINARY, OP_CONT):
                        message += payload
                        if len(message) > self.max_message:
                            self._send(conn, create_frame(struct.pack(">H", 1009), OP_CLOSE))
                            raise ConnectionAbortedError
                        if fin:
                            self._on_text(conn, message.decode("utf-8", "replace"))
                            message = b""
        except (OSError, ConnectionAbortedError):
            pass
        self._remove(conn)

    def _on_text(self, conn: socket.socket, text: str):
        if self.on_message is not None:
            self.on_message(text)
        if self.generate_cb is None:
            return
        try:
            req = json.loads(text)
            prompt, max_tokens = str(req["prompt"]), int(req.get("max_tokens", 64))
        except (ValueError, KeyError, TypeError):
            self._send(conn, create_frame(json.dumps({"error": "expected {\"prompt\": ..., \"max_tokens\": ...}"})))
            return
        out = self.generate_cb(prompt, max_tokens, True)
        for piece in ([out] if isinstance(out, str) else out):
            self._send(conn, create_frame(piece))
        self._send(conn, create_frame(json.dumps({"done": True})))

    def _remove(self, conn: socket.socket):
        with self._lock:
            if conn in self._clients:
                self._clients.remove(conn)
            self._send_locks.pop(conn, None)
        self._close(conn)

    @staticmethod
    def _close(conn: socket.socket):
        try:
            conn.close()
        except OSError:
            pass


class WebSocketClient:
    """Minimal client (masked frames) for tests and the command-line tools."""

    def __init__(self, host: str, port: int, timeout: float = 5.0):
        self.sock = socket.create_connection((host, port), timeout=timeout)
        key = base64.b64encode(b"innova-b200-client").decode()
        self.sock.sendall((f"GET / HTTP/1.1\r\nHost: {host}:{port}\r\nUpgrade: websocket\r\nConnection: Upgrade\r\n"
                           f"Sec-WebSocket-Key: {key}\r\nSec-WebSocket-Version: 13\r\n\r\n").encode())
        data = b""
        while b"\r\n\r\n" not in data:
            chunk = self.sock.recv(4096)
            if not chunk:
                raise ConnectionError("handshake closed")
            data += chunk
        head, self._buf = data.split(b"\r\n\r\n", 1)
        if b" 101 " not in head.split(b"\r\n")[0] or compute_accept_key(key).encode() not in head:
            raise ConnectionError("handshake refused")

    def send(self, data: Union[str, bytes], opcode: int = OP_TEXT):
        self.sock.sendall(create_frame(data, opcode, mask=b"\x12\x34\x56\x78"))

    def recv(self) -> Tuple[int, bytes]:
        while True:
            fr = parse_frame(self._buf)
            if fr is not None:
                payload, op, _, used = fr
                self._buf = self._buf[used:]
                return op, payload
            chunk = self.sock.recv(65536)
            if not chunk:
                raise ConnectionError("closed")
            self._buf += chunk

    def close(self):
        try:
            self.send(struct.pack(">H", 1000), OP_CLOSE)
        except OSError:
            pass
        self.sock.close()
