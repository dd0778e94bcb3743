"""Inter-stage communication with the reference handler's interface and routing.

`CommunicationHandler` keeps the constructor, `initialize`, `set_tensor_shapes`,
`start_helper_threads`, `send`, `recv`, `increment_messaging_index` and `wait`
of runtime/communication.py:18-608, and reproduces its routing arithmetic
exactly (forward sends and backward receives round-robin over the next stage's
replicas, :583-608; forward receives and backward sends follow the messaging
schedule, :456-521).  What moves the bytes is different: there are no helper
threads, no host staging and no shape messages over TCP.  A transport delivers
each (tensor, peer, direction) FIFO:

  "p2p" / "nccl" : one process per GPU; the producer copies the payload over
                   NVLink into a ring slot in the consumer's HBM (CUDA IPC) on a
                   side stream and publishes a sequence flag (peer_channel.py)
  "local"        : every stage of a pipeline in one process on one GPU (a way to
                   run a multi-stage configuration on a single device); tensors
                   are handed over by reference

Other names are refused unless a transport was registered for them with
`register_transport` (the CPU tests of the host logic register one over gloo).
"""
import collections
import os
import threading

import torch
import torch.distributed as dist

NCCL = 'nccl'
GLOO = 'gloo'
LOCAL = 'local'
P2P = 'p2p'


# --------------------------------------------------------------------------- #
# routing arithmetic (pure Python, shared by every transport)
# --------------------------------------------------------------------------- #
class MessagingSchedule:
    """Order in which a replica receives forward tensors from, and sends gradients
    to, the replicas of the previous stage (runtime/communication.py:456-521)."""

    def __init__(self, rank_in_stage, num_ranks_in_stage, num_ranks_in_previous_stage):
        self.rows = []
        for i in range(num_ranks_in_stage):
            row = list(range(i, num_ranks_in_previous_stage, num_ranks_in_stage))
            if row:
                self.rows.append(row)
        self.fwd_row = self.bwd_row = rank_in_stage
        self.fwd_col = self.bwd_col = 0
        # previous stage has fewer replicas than this one
        while self.rows and self.fwd_row >= len(self.rows):
            self.fwd_row -= 1
            self.bwd_row -= 1

    def index(self, sending):
        if sending:
            return self.rows[self.bwd_row][self.bwd_col]
        return self.rows[self.fwd_row][self.fwd_col]

    def increment(self, sending):
        if sending:
            self.bwd_col += 1
            if self.bwd_col == len(self.rows[self.bwd_row]):
                self.bwd_col = 0
                self.bwd_row -= 1
                if self.bwd_row == -1:
                    self.bwd_row = len(self.rows) - 1
        else:
            self.fwd_col += 1
            if self.fwd_col == len(self.rows[self.fwd_row]):
                self.fwd_col = 0
                self.fwd_row -= 1
                if self.fwd_row == -1:
                    self.fwd_row = len(self.rows) - 1


def forward_send_index(forward_minibatch_id, rank_in_stage, num_next):
    """Replica of the next stage that gets this minibatch (runtime/communication.py:606-608)."""
    return (forward_minibatch_id + rank_in_stage) % num_next


def backward_recv_index(backward_minibatch_id, rank_in_stage, num_next):
    """Replica of the next stage whose gradient is consumed (runtime/communication.py:586-590)."""
    return (backward_minibatch_id + rank_in_stage) % num_next


# --------------------------------------------------------------------------- #
# transports
# --------------------------------------------------------------------------- #
class _LocalFabric:
    """In-process FIFOs keyed by (src_rank, dst_rank, tensor_name, backward)."""

    def __init__(self):
        self.queues = collections.defaultdict(collections.deque)
        self.lock = threading.Lock()

    def put(self, key, tensor):
        with self.lock:
            self.queues[key].append(tensor)

    def ready(self, key):
        return len(self.queues[key]) > 0

    def get(self, key):
        with self.lock:
            if not self.queues[key]:
                raise RuntimeError("local fabric: nothing queued for %r (schedule error)" % (key,))
            return self.queues[key].popleft()


LOCAL_FABRIC = _LocalFabric()


def reset_local_fabric():
    LOCAL_FABRIC.queues.clear()


class _LocalTransport:
    def __init__(self, rank):
        self.rank = rank

    def send(self, dst_rank, name, backward, tensor, tag):
        LOCAL_FABRIC.put((self.rank, dst_rank, name, backward), tensor.detach())

    def recv(self, src_rank, name, backward, shape, dtype, tag):
        return LOCAL_FABRIC.get((src_rank, self.rank, name, backward))

    def ready(self, src_rank, name, backward):
        return LOCAL_FABRIC.ready((src_rank, self.rank, name, backward))

    def wait(self):
        pass


TRANSPORTS = {}      # backend name -> factory(handler, master_addr, master_port) returning a transport


def register_transport(name, factory):
    """Adds a backend.  factory(handler, master_addr, master_port) is called from the handler's constructor and
    returns an object with send(dst_rank, name, backward, tensor, tag), recv(src_rank, name, backward, shape,
    dtype, tag) and wait(); `uses_process_groups` (default True) says whether torch.distributed groups exist."""
    TRANSPORTS[name] = factory


def _rendezvous_env(master_addr, master_port):
    """MASTER_ADDR / MASTER_PORT as the reference sets them (runtime/communication.py:38-40),
    unless a launcher (torch.distributed.run) already hosts the rendezvous store."""
    if os.environ.get("TORCHELASTIC_RUN_ID") or os.environ.get("TORCHELASTIC_USE_AGENT_STORE"):
        return
    os.environ['MASTER_ADDR'] = master_addr
    os.environ['MASTER_PORT'] = str(master_port)


# --------------------------------------------------------------------------- #
# handler
# --------------------------------------------------------------------------- #
class CommunicationHandler(object):
    """Handles communication between stages (interface of runtime/communication.py:18)."""

    def __init__(self, master_addr, master_port, rank, local_rank, num_ranks_in_server,
                 world_size, fp16, backend):
        self.rank = rank
        self.local_rank = local_rank
        self.backend = backend
        self.num_ranks_in_server = num_ranks_in_server
        self.world_size = world_size
        self.fp16 = fp16
        # Translation batches change their sequence length every minibatch; the reference sends the
        # shape ahead of every payload (runtime/communication.py:664-669).  Here the shape rides in the
        # slot header and is only read back (a host wait) when this flag is set by the runtime.
        self.variable_shapes = False
        assert num_ranks_in_server > 0
        if backend == LOCAL:
            self.transport = _LocalTransport(rank)
        elif backend in (NCCL, P2P):
            from . import peer_channel
            if not dist.is_initialized():
                _rendezvous_env(master_addr, master_port)
                dist.init_process_group(NCCL, rank=rank, world_size=world_size,
                                        device_id=torch.device("cuda", local_rank))
            assert dist.get_world_size() == self.world_size
            self.transport = peer_channel.PeerTransport(rank, world_size, local_rank)
        elif backend in TRANSPORTS:
            self.transport = TRANSPORTS[backend](self, master_addr, master_port)
        else:
            raise ValueError("distributed backend %r is not available: boundary tensors move over NVLink peer "
                             "channels (\"p2p\" or \"nccl\") or inside one process (\"local\")" % (backend,))
        self.gradient_tensor_names = None

    def uses_process_groups(self):
        return self.backend != LOCAL and getattr(self.transport, "uses_process_groups", True)

    def initialize(self, receive_ranks, send_ranks, tensor_tags, target_tensor_names,
                   training_tensor_dtypes, rank_in_stage, num_ranks_in_stage,
                   ranks_in_previous_stage, ranks_in_next_stage):
        self.receive_ranks = receive_ranks
        self.send_ranks = send_ranks
        self.tensor_tags = tensor_tags
        self.target_tensor_names = target_tensor_names
        self.training_tensor_dtypes = training_tensor_dtypes
        self.rank_in_stage = rank_in_stage
        self.num_ranks_in_stage = num_ranks_in_stage
        self.ranks_in_previous_stage = ranks_in_previous_stage
        self.num_ranks_in_previous_stage = len(ranks_in_previous_stage)
        self.ranks_in_next_stage = ranks_in_next_stage
        self.num_ranks_in_next_stage = len(ranks_in_next_stage)
        # Targets travel with the activations to every later stage: the reference adds them
        # to the (shared) rank dictionaries here (runtime/communication.py:165-188).
        for name in self.target_tensor_names:
            if self.num_ranks_in_previous_stage > 0:
                self.receive_ranks[name] = self.ranks_in_previous_stage
            if self.num_ranks_in_next_stage > 0:
                self.send_ranks[name] = self.ranks_in_next_stage
        self.setup_messaging_schedule()
        self.tensor_shapes = None
        self.forward_only = False

    def setup_messaging_schedule(self):
        self.schedule = MessagingSchedule(self.rank_in_stage, self.num_ranks_in_stage,
                                          self.num_ranks_in_previous_stage)
        self.messaging_schedule = self.schedule.rows

    def get_messaging_index(self, sending):
        return self.schedule.index(sending)

    def increment_messaging_index(self, sending):
        self.schedule.increment(sending)

    def set_tensor_shapes(self, tensor_shapes):
        self.tensor_shapes = tensor_shapes

    def num_iterations_for_helper_threads(self, num_iterations):
        """Per-peer message counts (runtime/communication.py:222-248); uneven splits are rejected."""
        fwd = bwd = num_iterations
        if self.num_ranks_in_next_stage > 0:
            assert fwd % self.num_ranks_in_next_stage == 0
            fwd //= self.num_ranks_in_next_stage
        else:
            fwd = 0
        if self.num_ranks_in_previous_stage > 0:
            assert bwd % self.num_ranks_in_previous_stage == 0
            bwd //= self.num_ranks_in_previous_stage
        else:
            bwd = 0
        return fwd, bwd

    def start_helper_threads(self, num_iterations, forward_only):
        """Start of an epoch.  Nothing is spawned; "ack" joins the rank maps for forward-only
        runs exactly as in the reference (runtime/communication.py:254-267)."""
        self.forward_only = forward_only
        if forward_only:
            self.receive_ranks["ack"] = self.ranks_in_previous_stage
            self.send_ranks["ack"] = self.ranks_in_next_stage
        else:
            self.receive_ranks.pop("ack", None)
            self.send_ranks.pop("ack", None)
        self.num_iterations_for_helper_threads(num_iterations)
        if hasattr(self.transport, "setup"):
            self.transport.setup(self, self.tensor_shapes)    # collective: opens missing peer channels

    def wait(self):
        self.transport.wait()

    # ------------------------------------------------------------------ data path
    def _dtype(self, name):
        """Element type of a boundary tensor on the wire.  The driver scripts record the dtypes from a dry run
        of the fp32 CPU model (main_with_runtime.py:139-155), so with `fp16` every floating tensor is really
        the 16-bit compute type - the reference makes the same substitution (runtime/communication.py:273)."""
        if name == "ack":
            return torch.int64
        dtype = self.training_tensor_dtypes.get(name)
        if dtype is None:
            return torch.int64          # targets without a recorded dtype (runtime/communication.py:320)
        if self.fp16 and dtype.is_floating_point:
            return torch.bfloat16
        return dtype

    def recv(self, tensor_name, forward_minibatch_id, backward_minibatch_id, backward=False):
        if backward:
            peers = self.send_ranks[tensor_name]
            index = backward_recv_index(backward_minibatch_id, self.rank_in_stage, len(peers))
        else:
            peers = self.receive_ranks[tensor_name]
            index = self.get_messaging_index(sending=False)
        tensor = self.transport.recv(peers[index], tensor_name, backward,
                                     self.tensor_shapes[tensor_name], self._dtype(tensor_name),
                                     self.tensor_tags[tensor_name])
        if not backward and tensor.is_floating_point():
            tensor = tensor.requires_grad_()
        return tensor

    def send(self, tensor_name, tensor, forward_minibatch_id, backward_minibatch_id, backward=False):
        if backward:
            peers = self.receive_ranks[tensor_name]
            index = self.get_messaging_index(sending=True)
        else:
            peers = self.send_ranks[tensor_name]
            index = forward_send_index(forward_minibatch_id, self.rank_in_stage, len(peers))
        self.transport.send(peers[index], tensor_name, backward, tensor, self.tensor_tags[tensor_name])

    # ------------------------------------------------------------------ readiness (local transport)
    def forward_ready(self):
        """True when every forward input of the next minibatch has arrived (local transport only)."""
        for name, peers in self.receive_ranks.items():
            if name == "ack":
                continue
            if not self.transport.ready(peers[self.get_messaging_index(sending=False)], name, False):
                return False
        return True

    def backward_ready(self, backward_minibatch_id):
        for name, peers in self.send_ranks.items():
            if name in self.target_tensor_names or name == "ack":
                continue
            if self.gradient_tensor_names is not None and name not in self.gradient_tensor_names:
                continue
            idx = backward_recv_index(backward_minibatch_id, self.rank_in_stage, len(peers))
            if not self.transport.ready(peers[idx], name, True):
                return False
        return True
