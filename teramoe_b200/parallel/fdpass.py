"""File descriptors between the ranks of one node, over Unix sockets.

A memory allocation made with the driver's virtual memory management is shared with other processes as a POSIX file
descriptor, and a descriptor only means something inside the process that owns it: it has to travel as `SCM_RIGHTS`
ancillary data over a Unix-domain socket.  ``exchange_fds`` is the collective that does it: every rank hands in one
descriptor and gets back one (received, process-local) descriptor per peer.

How: every rank listens on an abstract-namespace socket (no file system entry, gone with the process), the names go
round through the process group (which also orders "everyone listens" before "anyone connects"), every rank connects to
every peer, accepts its peers' connections, says who it is on each and sends its descriptor; then it reads the
descriptor of each peer from the connection it opened to it.  The backlog holds all connections, so no rank needs a
thread.

Reference counterpart: the fabric / POSIX-handle exchange of shared_memory::SharedMemoryAllocator and
Buffer::sync (csrc/moe_extension.cpp:16-125, :291-436), which passes handles as bytes through the process group; a
descriptor cannot go that way.
"""
from __future__ import annotations

import os
import socket
import struct
import uuid
from typing import List, Optional

import torch.distributed as dist

_TIMEOUT_S = 60.0


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = b""
    while len(buf) < n:
        part = sock.recv(n - len(buf))
        if not part:
            raise RuntimeError("teramoe_b200: peer closed the descriptor socket early")
        buf += part
    return buf


def exchange_fds(fd: int, rank: int, size: int, group=None, gather=None) -> List[int]:
    """Collective: returns ``fds`` with ``fds[r]`` = this process's copy of rank r's descriptor (``fds[rank] = fd``).

    The caller owns the returned descriptors of the peers (close them, or hand them to an importer that does).
    ``gather`` replaces the process-group all-gather of the socket names (tests).
    """
    if size == 1:
        return [fd]
    name = b"\0teramoe_b200_fd_" + uuid.uuid4().hex.encode() + b"_%d_%d" % (os.getpid(), rank)
    listener = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    conns: List[Optional[socket.socket]] = [None] * size
    out = [-1] * size
    out[rank] = fd
    try:
        listener.bind(name)
        listener.listen(size + 4)
        listener.settimeout(_TIMEOUT_S)
        if gather is not None:
            names = gather(name)
        else:
            names = [None] * size
            dist.all_gather_object(names, name, group=group)
        if any(not isinstance(n, (bytes, bytearray)) for n in names) or len(names) != size:
            raise RuntimeError("teramoe_b200: malformed socket name received during the descriptor exchange")
        for r in range(size):
            if r == rank:
                continue
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.settimeout(_TIMEOUT_S)
            c.connect(bytes(names[r]))
            c.sendall(struct.pack("<i", rank))
            conns[r] = c
        for _ in range(size - 1):
            a, _addr = listener.accept()
            try:
                a.settimeout(_TIMEOUT_S)
                # the socket name is unguessable, but an allocation is only ever handed to a process of the same user
                _pid, uid, _gid = struct.unpack("3i", a.getsockopt(socket.SOL_SOCKET, socket.SO_PEERCRED, struct.calcsize("3i")))
                if uid != os.getuid():
                    raise RuntimeError(f"teramoe_b200: descriptor requested by a process of another user (uid {uid})")
                (peer,) = struct.unpack("<i", _recv_exact(a, 4))
                if not (0 <= peer < size) or peer == rank:
                    raise RuntimeError(f"teramoe_b200: descriptor requested by an unknown rank {peer}")
                socket.send_fds(a, [b"F"], [fd])
            finally:
                a.close()
        for r in range(size):
            if r == rank:
                continue
            msg, fds, _flags, _addr = socket.recv_fds(conns[r], 1, 1)
            if msg != b"F" or len(fds) != 1:
                for f in fds:
                    os.close(f)
                raise RuntimeError(f"teramoe_b200: no descriptor received from rank {r}")
            out[r] = fds[0]
        return out
    except BaseException:
        for r, f in enumerate(out):
            if r != rank and f >= 0:
                os.close(f)
        raise
    finally:
        for c in conns:
            if c is not None:
                c.close()
        listener.close()
