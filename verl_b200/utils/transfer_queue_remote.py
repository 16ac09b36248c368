"""TransferQueue over TCP: one process serves a ``TransferQueue``; any number of client processes (rollout workers, trainer
ranks, reward workers) use ``RemoteTransferQueue`` with the same methods as the in-process store.

Wire format: every message is an 8-byte big-endian length followed by a pickled ``(method, args, kwargs)`` request or a
pickled ``("ok", result)`` / ``("err", repr)`` reply; tensors travel as CPU tensors. One thread per connection; requests of a
connection are answered in order. ``wait_for_tags`` blocks on the server until a predicate over the partition's tags holds,
so clients do not poll. Pickle is only safe between trusted processes of one job: bind to 127.0.0.1 or a private interface.

Reference: the external TransferQueue service and its client used by ``verl/utils/transferqueue_utils.py:160-347``.
"""

from __future__ import annotations

import pickle
import socket
import socketserver
import struct
import threading
from typing import Iterable, Optional

from verl_b200.protocol import DataProto
from verl_b200.utils.transfer_queue import KVBatchMeta, TransferQueue

__all__ = ["TransferQueueServer", "RemoteTransferQueue"]

_METHODS = {"kv_put", "kv_batch_put", "kv_clear", "kv_tags", "kv_get", "size", "wait_for_tags"}


def _send(sock: socket.socket, obj) -> None:
    payload = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    sock.sendall(struct.pack(">Q", len(payload)) + payload)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(min(n - len(buf), 1 << 20))
        if not chunk:
            raise ConnectionError("transfer queue peer closed the connection")
        buf += chunk
    return bytes(buf)


def _recv(sock: socket.socket):
    (n,) = struct.unpack(">Q", _recv_exact(sock, 8))
    return pickle.loads(_recv_exact(sock, n))


def _tags_predicate(tags: dict, count: int, where: dict) -> bool:
    return sum(1 for t in tags.values() if all(t.get(k) == v for k, v in where.items())) >= count


class TransferQueueServer:
    """Serves ``queue`` (a new ``TransferQueue`` by default) on ``host:port`` (port 0 = any free port) in background threads."""

    def __init__(self, queue: Optional[TransferQueue] = None, host: str = "127.0.0.1", port: int = 0):
        self.queue = queue or TransferQueue()
        outer = self

        class Handler(socketserver.BaseRequestHandler):
            def handle(self):
                sock = self.request
                sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                while True:
                    try:
                        method, args, kwargs = _recv(sock)
                    except (ConnectionError, OSError, EOFError):
                        return
                    try:
                        if method not in _METHODS:
                            raise AttributeError(f"unknown transfer queue method {method!r}")
                        if method == "wait_for_tags":
                            result = outer._wait_for_tags(*args, **kwargs)
                        else:
                            result = getattr(outer.queue, method)(*args, **kwargs)
                        reply = ("ok", result)
                    except Exception as e:  # noqa: BLE001 - reported to the caller
                        reply = ("err", repr(e))
                    try:
                        _send(sock, reply)
                    except OSError:
                        return

        class Server(socketserver.ThreadingTCPServer):
            allow_reuse_address = True
            daemon_threads = True

        self._server = Server((host, port), Handler)
        self.address = f"{host}:{self._server.server_address[1]}"
        self._thread = threading.Thread(target=self._server.serve_forever, name="transfer-queue-server", daemon=True)
        self._thread.start()

    def _wait_for_tags(self, partition_id: str, count: int, where: dict, timeout: Optional[float] = None) -> bool:
        q = self.queue
        return q.wait(lambda: _tags_predicate(q._tags.get(partition_id, {}), count, where), timeout)

    def shutdown(self):
        self._server.shutdown()
        self._server.server_close()


class RemoteTransferQueue:
    """Client with the interface of ``TransferQueue`` (``kv_put / kv_batch_put / kv_clear / kv_tags / kv_get / size``) plus
    ``wait_for_tags``. Thread-safe: calls are serialised on one connection."""

    def __init__(self, address: str, timeout: Optional[float] = None):
        host, port = address.rsplit(":", 1)
        self._sock = socket.create_connection((host, int(port)), timeout=timeout)
        self._sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._lock = threading.Lock()

    def _call(self, method: str, *args, **kwargs):
        with self._lock:
            _send(self._sock, (method, args, kwargs))
            status, result = _recv(self._sock)
        if status != "ok":
            raise RuntimeError(f"transfer queue server: {result}")
        return result

    def kv_put(self, partition_id: str, key: str, fields: Optional[dict] = None, tags: Optional[dict] = None):
        return self._call("kv_put", partition_id, key, fields, tags)

    def kv_batch_put(self, meta: KVBatchMeta, data: DataProto, tags: Optional[dict] = None):
        return self._call("kv_batch_put", meta, data, tags)

    def kv_clear(self, partition_id: str, keys: Optional[Iterable[str]] = None):
        return self._call("kv_clear", partition_id, list(keys) if keys is not None else None)

    def kv_tags(self, partition_id: str) -> dict:
        return self._call("kv_tags", partition_id)

    def kv_get(self, meta: KVBatchMeta) -> DataProto:
        return self._call("kv_get", meta)

    def size(self, partition_id: str) -> int:
        return self._call("size", partition_id)

    def wait_for_tags(self, partition_id: str, count: int, where: dict, timeout: Optional[float] = None) -> bool:
        """Block (on the server) until at least ``count`` keys of the partition carry all ``where`` tag values."""
        return self._call("wait_for_tags", partition_id, count, where, timeout)

    def wait(self, predicate, timeout: Optional[float] = None) -> bool:
        """Polling fallback for arbitrary local predicates (closures cannot travel to the server)."""
        import time

        t0 = time.time()
        while not predicate():
            if timeout is not None and time.time() - t0 > timeout:
                return False
            time.sleep(0.01)
        return True

    def close(self):
        try:
            self._sock.close()
        except OSError:
            pass
