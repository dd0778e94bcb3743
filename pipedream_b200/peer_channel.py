"""NVLink peer-to-peer transport for CommunicationHandler: one process per GPU.

For every directed edge (producer rank, consumer rank, tensor, direction) the consumer owns a
ring of slots in its own HBM (`pd_chan_create`), the producer maps it with CUDA IPC
(`pd_chan_open`) and pushes payloads into it on a side stream; the consumer's side stream
waits for the sequence flag, copies the payload out and frees the slot.  The compute stream
only ever waits on events, the host never blocks on the data path, and every device-side wait
is bounded (a peer that is gone turns into an error status, not a hang).

This replaces the helper threads, queues and host staging of the reference's
runtime/communication.py:114-211,250-356,610-712.  Handles are exchanged once, when the tensor
shapes become known, through torch.distributed's object all-gather.
"""
import ctypes

import torch
import torch.distributed as dist

from . import _lib
from ._lib import call


def _nbytes(shape, dtype):
    n = 1
    for s in shape:
        n *= int(s)
    return n * torch.empty((), dtype=dtype).element_size()


class PeerTransport:
    def __init__(self, rank, world_size, local_rank, timeout_ms=120000, num_slots=4):
        self.rank, self.world_size, self.local_rank = rank, world_size, local_rank
        self.timeout_ms, self.num_slots = timeout_ms, num_slots
        self.device = torch.device("cuda", local_rank)
        self.consumers = {}      # key -> channel handle (this rank receives)
        self.producers = {}      # key -> channel handle (this rank sends)
        self.capacity = {}
        self.streams = {}
        self.keepalive = []
        self.variable_shapes = False
        _lib.load()

    def _stream(self, kind):
        s = self.streams.get(kind)
        if s is None:
            s = torch.cuda.Stream(device=self.device)
            self.streams[kind] = s
        return s

    # ------------------------------------------------------------------ set-up
    def _edges(self, h, shapes):
        """Edges this rank consumes: {(src, dst, name, backward): capacity in bytes}."""
        me, out = self.rank, {}
        for name, srcs in h.receive_ranks.items():
            if name not in shapes:
                continue
            for src in srcs:
                out[(src, me, name, 0)] = _nbytes(shapes[name], h._dtype(name))
        for name, srcs in h.send_ranks.items():
            if name in h.target_tensor_names or name not in shapes:
                continue
            for src in srcs:
                out[(src, me, name, 1)] = _nbytes(shapes[name], h._dtype(name))
        return out

    def setup(self, handler, shapes):
        """Create the rings this rank consumes, exchange their handles, map the ones it feeds.
        Collective: every rank calls it at the same points (StageRuntime.train / eval)."""
        torch.cuda.set_device(self.device)
        self.variable_shapes = bool(getattr(handler, "variable_shapes", False))
        need = self._edges(handler, shapes)
        blobs = {}
        for key, cap in need.items():
            if key in self.consumers and self.capacity[key] >= cap:
                continue
            if key in self.consumers:
                raise _lib.PipedreamB200Error("peer channel %r would need to grow from %d to %d bytes; "
                                              "open it with the largest shapes first" % (key, self.capacity[key], cap))
            ch = ctypes.c_void_p()
            call("pd_chan_create", cap, self.num_slots, self.timeout_ms, ctypes.byref(ch))
            blob = ctypes.create_string_buffer(128)
            call("pd_chan_export_handle", ch, blob)
            self.consumers[key] = ch
            self.capacity[key] = cap
            blobs[key] = blob.raw
        gathered = [None] * self.world_size
        dist.all_gather_object(gathered, blobs)
        for peer_blobs in gathered:
            for key, raw in peer_blobs.items():
                if key[0] != self.rank or key in self.producers:
                    continue
                ch = ctypes.c_void_p()
                call("pd_chan_open", ctypes.create_string_buffer(raw, 128), self.timeout_ms, ctypes.byref(ch))
                self.producers[key] = ch
        dist.barrier()

    # ------------------------------------------------------------------ data path
    def send(self, dst_rank, name, backward, tensor, tag):
        key = (self.rank, dst_rank, name, 1 if backward else 0)
        ch = self.producers.get(key)
        if ch is None:
            raise _lib.PipedreamB200Error("no peer channel for %r (tensor shapes were not set?)" % (key,))
        t = tensor.detach()
        if not t.is_contiguous():
            from . import functional as pf
            pad = pf.padded_of(t)
            t = pf.unpack_pnhwc(pad) if pad is not None else t.contiguous()
        self._poll(key, ch)
        cur = torch.cuda.current_stream(self.device)
        side = self._stream("send_bwd" if backward else "send_fwd")
        ev = torch.cuda.Event()
        ev.record(cur)
        side.wait_event(ev)
        dims = (ctypes.c_int64 * max(1, t.dim()))(*t.shape)
        call("pd_chan_push", ch, ctypes.c_void_p(t.data_ptr()), t.numel() * t.element_size(), t.dim(), dims,
             ctypes.c_void_p(side.cuda_stream))
        t.record_stream(side)

    def recv(self, src_rank, name, backward, shape, dtype, tag):
        key = (src_rank, self.rank, name, 1 if backward else 0)
        ch = self.consumers.get(key)
        if ch is None:
            raise _lib.PipedreamB200Error("no peer channel for %r (tensor shapes were not set?)" % (key,))
        self._poll(key, ch)
        cur = torch.cuda.current_stream(self.device)
        side = self._stream("recv_bwd" if backward else "recv_fwd")
        if self.variable_shapes:
            # wait (on the host) for the message and take its shape from the slot header
            hdr = (ctypes.c_int64 * 8)()
            call("pd_chan_peek_header", ch, hdr, ctypes.c_void_p(side.cuda_stream))
            shape = tuple(int(hdr[3 + i]) for i in range(int(hdr[2])))
        out = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        ev = torch.cuda.Event()
        ev.record(cur)
        side.wait_event(ev)          # `out` may reuse memory still read by queued compute kernels
        call("pd_chan_wait", ch, ctypes.c_void_p(out.data_ptr()), out.numel() * out.element_size(),
             ctypes.c_void_p(side.cuda_stream))
        done = torch.cuda.Event()
        done.record(side)
        cur.wait_event(done)
        out.record_stream(side)
        return out

    def _poll(self, key, ch):
        """Raises as soon as an earlier operation on this channel has failed on the device (a wait that ran
        out, a message of the wrong size).  Reads a pinned host word: no stream is synchronised."""
        if _lib.load().pd_chan_poll(ch) != 0:
            raise _lib.PipedreamB200Error("peer channel %r: %s" % (key, _lib.last_error()))

    def wait(self):
        """End of an epoch: drain the side streams and surface any wait that ran out."""
        for s in self.streams.values():
            s.synchronize()
        self.check()

    def check(self):
        cur = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        for table in (self.consumers, self.producers):
            for key, ch in table.items():
                rc = _lib.load().pd_chan_status(ch, cur)
                if rc != 0:
                    raise _lib.PipedreamB200Error("peer channel %r: %s" % (key, _lib.last_error()))

    def close(self):
        for table in (self.producers, self.consumers):
            for ch in table.values():
                _lib.load().pd_chan_close(ch)
            table.clear()
