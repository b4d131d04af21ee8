"""Wire protocol v1, client side: big-endian, u32 body-length prefix, raw token ids.

Same functions and checks as the reference's server/protocol.py:5-40 (`request`, `cancellation`,
`decode_response`, `read_response`); the one difference is that a response may report a batch
size of up to 64, because this server batches up to 64 requests per GPU (the reference stops at 32).
"""
from __future__ import annotations

import struct

VERSION, GENERATE, CANCEL, FINAL, FIRST = 1, 1, 2, 0x8001, 0x8002
OK, INVALID, OVERLOADED, CANCELLED, INTERNAL = 0, 1, 2, 3, 4            # response status (server/include/protocol.hpp:33-45)
REQUEST = struct.Struct("!HHQII")
RESPONSE = struct.Struct("!HHQIIIIQQQQ")
MAX_RESPONSE = 60 + 4 * 1024
MAX_BATCH = 64
VOCAB = 50257


def _frame(body):
    return struct.pack("!I", len(body)) + body


def request(identifier, tokens, max_new_tokens):
    if type(identifier) is not int or not 0 < identifier < 2 ** 64:
        raise ValueError("request ID")
    if not tokens or any(type(t) is not int or not 0 <= t < VOCAB for t in tokens):
        raise ValueError("tokens")
    if type(max_new_tokens) is not int or max_new_tokens < 1 or len(tokens) + max_new_tokens > 1024:
        raise ValueError("context")
    return _frame(REQUEST.pack(VERSION, GENERATE, identifier, max_new_tokens, len(tokens)) + struct.pack(f"!{len(tokens)}I", *tokens))


def cancellation(identifier):
    if type(identifier) is not int or not 0 < identifier < 2 ** 64:
        raise ValueError("request ID")
    return _frame(REQUEST.pack(VERSION, CANCEL, identifier, 0, 0))


def decode_response(body):
    if len(body) < RESPONSE.size:
        raise ValueError("response size")
    version, kind, identifier, status, count, batch, reserved, queue, first, infer, total = RESPONSE.unpack_from(body)
    if (version != VERSION or kind not in (FIRST, FINAL) or not identifier or status not in range(5) or reserved
            or len(body) != RESPONSE.size + 4 * count):
        raise ValueError("response schema")
    if batch > MAX_BATCH or count > 1024 or (kind == FIRST and (status or count != 1)):
        raise ValueError("response bounds")
    tokens = list(struct.unpack_from(f"!{count}I", body, RESPONSE.size)) if count else []
    if any(t >= VOCAB for t in tokens):
        raise ValueError("response token")
    return {"kind": kind, "id": identifier, "status": status, "tokens": tokens, "batch_size": batch,
            "queue_ns": queue, "first_ns": first, "infer_ns": infer, "server_ns": total}


async def read_response(reader):
    size = struct.unpack("!I", await reader.readexactly(4))[0]
    if not RESPONSE.size <= size <= MAX_RESPONSE:
        raise ValueError("response frame limit")
    return decode_response(await reader.readexactly(size))


def recv_response(sock):
    """Blocking-socket variant of read_response."""
    def exactly(n):
        data = b""
        while len(data) < n:
            piece = sock.recv(n - len(data))
            if not piece:
                raise ConnectionError("server closed the connection")
            data += piece
        return data
    size = struct.unpack("!I", exactly(4))[0]
    if not RESPONSE.size <= size <= MAX_RESPONSE:
        raise ValueError("response frame limit")
    return decode_response(exactly(size))
