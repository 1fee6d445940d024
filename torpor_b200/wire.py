"""The remoting wire surface of the swap path, and an executor loop over it.

Torpor's clients reach the server with protobuf messages (proto/cudarpc.proto: ``QueryList``
of ``WapperQuery{type, query, client_id, need_sync}``; proto/signal.proto: ``SignalRequest`` /
``SignalAck``).  The swap engine must drop in behind that surface unchanged, so this module
speaks it: a small proto3 codec for exactly the messages that touch memory (field numbers
and types as in cudarpc.proto:74-83,300-353,400-415 and signal.proto:15-29 -- ``protoc`` is
not needed), and ``WireExecutor``, which does for those messages what the reference's
``CUDAExecutor`` does (include/server/cuda_server.hpp:212-255,951-1065,1226-1310): malloc /
memcpy / memset / synchronize are forwarded to the memory manager, and ``cudaLaunchKernel``
records on the first run which 8-byte argument words hold model pointers and rewrites exactly
those words through ``get_cuda_addr`` afterwards.  Kernels are not launched here -- the
rewritten argument list is returned -- because only the swap path is under test.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple

# QueryType values (proto/cudarpc.proto:7-50)
Q_DEVICE_SYNCHRONIZE, Q_MALLOC, Q_FREE, Q_MEMCPY, Q_MEMCPY_ASYNC, Q_MEMSET_ASYNC, Q_LAUNCH_KERNEL = 14, 30, 31, 32, 33, 34, 50
Q_STREAM_SYNCHRONIZE = 23
# cudaMemcpyKind
H2D, D2H, D2D = 1, 2, 3
# signal.RequestType (proto/signal.proto:5-13) and executor signals (common/include/utils.hpp:70-74)
REQ_EXECUTE_AFTER_LOAD, REQ_EXECUTE, REQ_LOAD, REQ_UNLOAD = 0, 1, 2, 3
SIG_NOTIFY, SIG_STARTUP, SIG_EXECUTE, SIG_UNLOAD, SIG_LOAD = 0, 1, 2, 3, 4

VARINT, LEN = 0, 2

# message -> [(field number, name, kind)]; kind: "u" varint, "b" bytes, "s" string, "rb" repeated bytes,
# "rm:<message>" repeated sub-message
SCHEMA: Dict[str, List[Tuple[int, str, str]]] = {
    "WapperQuery": [(1, "type", "u"), (2, "query", "b"), (3, "client_id", "u"), (4, "need_sync", "u")],
    "QueryList": [(1, "queries", "rm:WapperQuery")],
    "genericResponse": [(1, "error", "u")],
    "cudaMallocQuery": [(1, "size", "u")],
    "cudaMallocResponse": [(1, "error", "u"), (2, "ptr", "u")],
    "cudaFreeQuery": [(1, "ptr", "u")],
    "cudaMemcpyQuery": [(1, "kind", "u"), (2, "src", "u"), (3, "dst", "u"), (4, "count", "u"), (5, "payload", "b")],
    "cudaMemcpyResponse": [(1, "error", "u"), (2, "payload", "b")],
    "cudaMemcpyAsyncQuery": [(1, "kind", "u"), (2, "src", "u"), (3, "dst", "u"), (4, "count", "u"), (5, "payload", "b"),
                             (6, "stream", "b")],
    "cudaMemcpyAsyncResponse": [(1, "ptr", "u"), (2, "payload", "b")],
    "AsyncResponse": [(1, "error", "u"), (2, "responses", "rm:cudaMemcpyAsyncResponse")],
    "cudaMemsetAsyncQuery": [(1, "ptr", "u"), (2, "value", "u"), (3, "count", "u"), (4, "stream", "b")],
    "cudaLaunchKernelQuery": [(1, "function", "s"), (2, "grid_dim_x", "u"), (3, "grid_dim_y", "u"), (4, "grid_dim_z", "u"),
                              (5, "block_dim_x", "u"), (6, "block_dim_y", "u"), (7, "block_dim_z", "u"), (8, "args", "rb"),
                              (9, "shared_mem", "u"), (10, "stream", "b")],
    "SignalRequest": [(1, "type", "u"), (2, "function", "s"), (3, "payload", "s")],
    "SignalAck": [(1, "ack", "u"), (2, "resp", "u")],
}


def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1          # negative int32 travel as 10-byte varints, like protobuf
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    shift = val = 0
    while True:
        if pos >= len(buf):
            raise ValueError("truncated varint")
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, pos
        shift += 7
        if shift > 70:
            raise ValueError("varint too long")


def encode(message: str, fields: dict) -> bytes:
    """Serialise like protobuf's proto3: fields in number order, defaults omitted."""
    out = bytearray()
    for num, name, kind in SCHEMA[message]:
        v = fields.get(name)
        if kind == "u":
            v = int(v or 0)
            if v:
                out += _varint(num << 3 | VARINT) + _varint(v)
        elif kind in ("b", "s"):
            data = (v or b"")
            data = data.encode() if isinstance(data, str) else bytes(data)
            if data:
                out += _varint(num << 3 | LEN) + _varint(len(data)) + data
        elif kind == "rb":
            for item in v or []:
                out += _varint(num << 3 | LEN) + _varint(len(item)) + bytes(item)
        elif kind.startswith("rm:"):
            for item in v or []:
                sub = item if isinstance(item, (bytes, bytearray)) else encode(kind[3:], item)
                out += _varint(num << 3 | LEN) + _varint(len(sub)) + sub
    return bytes(out)


def decode(message: str, buf: bytes) -> dict:
    spec = {num: (name, kind) for num, name, kind in SCHEMA[message]}
    out: dict = {}
    for num, name, kind in SCHEMA[message]:
        out[name] = [] if kind[0] == "r" else (0 if kind == "u" else (b"" if kind == "b" else ""))
    pos = 0
    buf = bytes(buf)
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == VARINT:
            val, pos = _read_varint(buf, pos)
        elif wt == LEN:
            n, pos = _read_varint(buf, pos)
            if n > len(buf) - pos:
                raise ValueError("truncated message")
            val = buf[pos:pos + n]
            pos += n
        elif wt in (1, 5):
            n = 8 if wt == 1 else 4
            if n > len(buf) - pos:
                raise ValueError("truncated message")
            val, pos = buf[pos:pos + n], pos + n
        else:
            raise ValueError(f"unsupported wire type {wt}")
        if num not in spec:
            continue                # unknown fields are skipped, as protobuf does
        name, kind = spec[num]
        if (kind == "u") != (wt == VARINT) or (kind != "u" and wt != LEN):
            continue                # a known number with another wire type is an unknown field to protobuf, too
        if kind == "u":
            out[name] = val
        elif kind == "b":
            out[name] = bytes(val)
        elif kind == "s":
            try:
                out[name] = bytes(val).decode()
            except UnicodeDecodeError:
                raise ValueError(f"field {num} of {message} is not valid UTF-8") from None
        elif kind == "rb":
            out[name].append(bytes(val))
        else:
            out[name].append(decode(kind[3:], val))
    return out


def int32(v: int) -> int:
    """A varint field declared int32, as a Python int."""
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >> 63 else v


LOAD_NONE, LOAD_MODEL, LOAD_TRACK = 0, 1, 2     # LoadModelFlag_* of the executor


class WireExecutor:
    """One executor (one GPU) fed with serialised cudarpc / signal messages."""

    def __init__(self, manager):
        self.mm = manager
        self.active_func = ""
        self.flag = LOAD_NONE
        # kernel_model_access_loc (src/server/kernel_lookup.cpp): func -> kernel -> {(arg, word)}
        self.access_loc: Dict[str, Dict[str, set]] = {}
        self.launched: List[Tuple[str, List[bytes]]] = []
        # lookup() (src/server/kernel_lookup.cpp): kernel name -> launcher(args, grid, block, shared_mem).
        # A kernel registered here is really launched, on the argument words as rewritten below.
        self.kernels: Dict[str, object] = {}
        self.async_results: list = []        # stream_async_msg_: (client's destination, array being read into)

    # ---- signals from the controller (cuda_server.hpp:212-255)
    def signal(self, sig: int, func: str):
        if sig == SIG_STARTUP:
            self.active_func, self.flag = func, LOAD_MODEL
            self.mm.set_track_model_memory(func)
        elif sig == SIG_EXECUTE:
            self.active_func, self.flag = func, LOAD_NONE
        elif sig == SIG_UNLOAD:
            self.mm.evict_model(func)
        elif sig >= SIG_LOAD:
            src = sig - SIG_LOAD - 1
            self.mm.sig_trans_thread(func, src if (src >= 0 and src != self.mm.server_id) else -1)

    def complete(self):
        """send_complete_signal (cuda_server.hpp:287-299)."""
        if self.flag == LOAD_TRACK:
            self.flag = LOAD_NONE
            self.mm.unset_track_model_memory(self.active_func)
        self.active_func = ""

    # ---- API stream from the client
    def handle(self, query_list: bytes) -> List[bytes]:
        """Dispatch one serialised QueryList; returns the serialised responses of the calls that answer."""
        responses = []
        for q in decode("QueryList", query_list)["queries"]:
            r = self.dispatch(q["type"], q["query"])
            if r is not None:
                responses.append(r)
        return responses

    def dispatch(self, qtype: int, body: bytes):
        f = self.active_func
        if qtype == Q_MALLOC:
            q = decode("cudaMallocQuery", body)
            ptr = self.mm.cudaMallocBackend(q["size"], self.flag == LOAD_MODEL, f)
            return encode("cudaMallocResponse", {"error": 0, "ptr": ptr})
        if qtype == Q_FREE:
            self.mm.cudaFreeBackend(decode("cudaFreeQuery", body)["ptr"], f)
            return encode("genericResponse", {"error": 0})
        if qtype in (Q_MEMCPY, Q_MEMCPY_ASYNC):
            q = decode("cudaMemcpyAsyncQuery" if qtype == Q_MEMCPY_ASYNC else "cudaMemcpyQuery", body)
            kind = int32(q["kind"])
            if kind == H2D:
                import numpy as np
                rc = self.mm.cudaMemcpyAsyncBackendHtoD(q["dst"], np.frombuffer(q["payload"], dtype=np.uint8), 0,
                                                        self.flag == LOAD_MODEL, f)
                return encode("cudaMemcpyResponse", {"error": 0 if rc == 0 else 1}) if qtype == Q_MEMCPY else None
            if kind == D2H:
                data = self.mm.cudaMemcpyAsyncBackendDtoH(q["src"], q["count"], 0, f)
                if qtype == Q_MEMCPY_ASYNC:
                    # the result copy: kept until the client synchronises the stream, and it ends the
                    # request (cuda_server.hpp:1038-1049); nothing is answered now
                    self.async_results.append((q["dst"], data))      # read after the synchronise
                    self.complete()
                    return None
                self._device_sync()
                return encode("cudaMemcpyResponse", {"error": 0, "payload": data.tobytes()})
            if kind == D2D:
                self.mm.cudaMemcpyAsyncBackendDtoD(q["dst"], q["src"], q["count"], 0, f)
                return encode("cudaMemcpyResponse", {"error": 0}) if qtype == Q_MEMCPY else None
            return encode("cudaMemcpyResponse", {"error": 1})
        if qtype == Q_MEMSET_ASYNC:
            q = decode("cudaMemsetAsyncQuery", body)
            self.mm.cudaMemsetAsyncBackend(q["ptr"], int32(q["value"]), q["count"], 0, f)
            return None
        if qtype == Q_DEVICE_SYNCHRONIZE:
            self._device_sync()
            # the synchronize after model.cuda() marks the end of the model (cuda_server.hpp:951-962)
            self.flag = LOAD_TRACK
            self.mm.init_model_readiness(f)
            return encode("genericResponse", {"error": 0})
        if qtype == Q_STREAM_SYNCHRONIZE:
            # the body is the stream handle itself, not a message (cuda_server.hpp:1131-1148): every result
            # copy issued since the last synchronise travels back in one AsyncResponse
            self._device_sync()
            pending, self.async_results = self.async_results, []
            return encode("AsyncResponse", {"error": 0, "responses": [{"ptr": p, "payload": b.tobytes()} for p, b in pending]})
        if qtype == Q_LAUNCH_KERNEL:
            q = decode("cudaLaunchKernelQuery", body)
            args = self.rewrite_args(q["function"], q["args"])
            self.launched.append((q["function"], args))
            launcher = self.kernels.get(q["function"])
            if launcher is not None:                # cudaLaunchKernel(ptr, gridDim, blockDim, args, sharedMem, stream), :1302
                launcher(args, (q["grid_dim_x"], q["grid_dim_y"], q["grid_dim_z"]),
                         (q["block_dim_x"], q["block_dim_y"], q["block_dim_z"]), q["shared_mem"])
            return None
        raise ValueError(f"query type {qtype} is not part of the swap path")

    def _device_sync(self):
        if self.mm.device >= 0:
            import torch
            torch.cuda.synchronize(self.mm.device)

    def rewrite_args(self, kernel: str, args: List[bytes]) -> List[bytes]:
        """cudaLaunchKernelService (cuda_server.hpp:1226-1310): record or rewrite pointer words."""
        f = self.active_func
        words = [list(struct.unpack(f"<{len(a) // 8}Q", a)) if len(a) % 8 == 0 else None for a in args]
        loc = self.access_loc.setdefault(f, {}).setdefault(kernel, set())
        if self.flag == LOAD_TRACK:
            for i, w in enumerate(words):
                if w is None:
                    continue
                for j, v in enumerate(w):
                    if self.mm.is_model_address(f, v):
                        self.mm.try_insert_model_access(v)
                        loc.add((i, j))
                    elif self.mm.valid_memory_address(f, v):
                        loc.add((i, j))
        else:
            for i, j in sorted(loc):
                words[i][j] = self.mm.get_cuda_addr(f, words[i][j])
        return [struct.pack(f"<{len(w)}Q", *w) if w is not None else a for w, a in zip(words, args)]


class WireServer:
    """The GPU server at its two wire surfaces: the router's ``SignalRequest`` / ``SignalAck``
    (proto/signal.proto) handled by the library's controller, whose signals go to one
    ``WireExecutor`` per GPU, and the clients' ``QueryList`` streams handled by those executors
    (include/server/controller.hpp:125-264 with cuda_server.hpp:212-300).  An executor that ends a
    request reports it here, as the reference's does through ``controller_sync_queue``."""

    def __init__(self, managers, mem_limit_bytes: int, schedule_policy: str = "IA", evict_policy: str = "IA",
                 pcie_pairs=None, nvlink=None):
        from .memory_manager import Controller
        self.executors = [WireExecutor(m) for m in managers]
        self.ctrl = Controller(len(managers), mem_limit_bytes, schedule_policy, evict_policy, pcie_pairs, nvlink)
        self.sent: List[Tuple[int, int, str]] = []       # (gpu, signal, func) in the order they were sent

    def close(self):
        self.ctrl.close()

    def _carry_out(self, events) -> List[bytes]:
        acks = []
        for e in events:
            if e[0] == "S":
                self.sent.append((e[1], e[2], e[3]))
                self.executors[e[1]].signal(e[2], e[3])
            else:
                acks.append(encode("SignalAck", {"ack": e[1], "resp": e[2] & 0xFFFFFFFFFFFFFFFF}))
        return acks

    def request(self, signal_request: bytes) -> List[bytes]:
        """One serialised SignalRequest from the router; returns the serialised SignalAck, if one is due now
        (a request that has to wait for a GPU is acknowledged when it starts)."""
        r = decode("SignalRequest", signal_request)
        return self._carry_out(self.ctrl.request(r.get("type", 0), r.get("function", ""), r.get("payload", "")))

    def complete(self, gpu: int) -> List[bytes]:
        """Executor ``gpu`` finished its request: completion bookkeeping, then the next queued request."""
        self.executors[gpu].complete()
        return self._carry_out(self.ctrl.complete(gpu))
