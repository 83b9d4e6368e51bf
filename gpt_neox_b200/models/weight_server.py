"""Hand the live training weights to a co-located process (an inference / sampling engine on the same GPU)
without a copy: each rank listens on ``localhost:<base port + rank>`` and sends, per tensor of the state
dict, the CUDA-IPC description of its storage (megatron/model/weight_server.py:10-64).  CPU tensors (tests,
host-initialised models) are sent by value.

Because the engine keeps all parameters in a few flat buffers, consecutive tensors share one storage and
therefore one IPC handle; the receiver opens each handle once.
"""
from __future__ import annotations

import pickle
import socket
import struct
from typing import List, Union

import torch


def _send_msg(sock, obj):
    data = pickle.dumps(obj)
    sock.sendall(struct.pack("!Q", len(data)) + data)


def _recv_msg(sock):
    hdr = b""
    while len(hdr) < 8:
        c = sock.recv(8 - len(hdr))
        if not c:
            return None
        hdr += c
    n = struct.unpack("!Q", hdr)[0]
    buf = bytearray()
    while len(buf) < n:
        c = sock.recv(min(1 << 20, n - len(buf)))
        if not c:
            raise ConnectionError("peer closed the connection mid-message")
        buf += c
    return pickle.loads(bytes(buf))


def describe_tensor(key, t, end: bool):
    d = {"state_dict_key": key, "dtype": t.dtype, "tensor_size": tuple(t.shape), "tensor_stride": tuple(t.stride()),
         "tensor_offset": t.storage_offset(), "requires_grad": False, "end": end}
    if t.is_cuda:
        st = t.untyped_storage()
        (dev, handle, size_bytes, offset_bytes, ref_handle, ref_offset, ev_handle, ev_sync) = st._share_cuda_()
        d.update(storage_cls=type(st), storage_device=dev, storage_handle=handle, storage_size_bytes=size_bytes,
                 storage_offset_bytes=offset_bytes, ref_counter_handle=ref_handle, ref_counter_offset=ref_offset,
                 event_handle=ev_handle, event_sync_required=ev_sync)
    else:
        d["value"] = t.detach().clone()
    return d


def send_tensor(state_dict_key, data, sock, end: bool):
    _send_msg(sock, describe_tensor(state_dict_key, data, end))


def send_state_dict(state_dict, sock):
    keys = list(state_dict.keys())
    for i, k in enumerate(keys):
        send_tensor(k, state_dict[k], sock, i == len(keys) - 1)
        sock.recv(4096)                       # wait for the receiver's acknowledgement


def start_server(model, ports: Union[int, List[int]] = 6000, accept_timeout_s: float = None):
    """Blocks until one client connected and received the whole state dict."""
    rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
    port = ports + rank if isinstance(ports, int) else ports[rank]
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        s.bind(("localhost", port))
        s.listen(1)
        s.settimeout(accept_timeout_s)
        conn, _ = s.accept()
        with conn:
            send_state_dict(model.state_dict(), conn)


def receive_state_dict(port: int, host: str = "localhost"):
    """Client side: rebuild the tensors (zero-copy views of the server's memory for CUDA tensors)."""
    out = {}
    with socket.create_connection((host, port)) as s:
        while True:
            d = _recv_msg(s)
            if d is None:
                break
            if "value" in d:
                t = d["value"]
            else:
                st = d["storage_cls"]._new_shared_cuda(d["storage_device"], d["storage_handle"],
                                                       d["storage_size_bytes"], d["storage_offset_bytes"],
                                                       d["ref_counter_handle"], d["ref_counter_offset"],
                                                       d["event_handle"], d["event_sync_required"])
                t = torch.empty(0, dtype=d["dtype"], device=f"cuda:{d['storage_device']}")
                t.set_(st, d["tensor_offset"], d["tensor_size"], d["tensor_stride"])
            out[d["state_dict_key"]] = t
            s.sendall(b"ok")
            if d["end"]:
                break
    return out
