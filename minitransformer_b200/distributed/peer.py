"""Peer-memory exchange among the ranks of a tensor-parallel group on one NVSwitch node.

Takes the place of the userbuffer communicators behind the reference's `ub_overlap_ag` /
`ub_overlap_rs` flags (miniTransformer/module/linear.py:649-671): every rank maps the other
ranks' buffers (CUDA IPC) and the library's own kernels move the data over NVLink:
  * the per-tensor abs-max MAX-reduction and the barriers are one-warp flag exchanges,
  * the all-gather of quantized activations is a pull: each rank's quantize kernel writes its
    shard into its shared buffer and one copy kernel assembles the gathered tensors,
  * the reduce-scatter of bf16 partial sums starts inside the producing GEMM, whose epilogue
    stores every tile straight into the owning rank's staging buffer, and ends with a local sum.
Handles travel through the process group once per buffer (all_gather_object); everything
afterwards is stream-ordered device work, no host synchronisation.
"""
import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import _lib, kernels

_ARENA_MIN_BYTES = 64 << 20     # large enough to be an allocation of its own in torch's caching allocator
_ALIGN = 4096


class SharedBuffer:
    """A byte range that exists on every rank: `tensor` is this rank's own range (uint8),
    `ptrs[r]` the address of rank r's range as mapped into this process."""

    def __init__(self, tensor: torch.Tensor, ptrs: Sequence[int]):
        self.tensor, self.ptrs = tensor, list(ptrs)
        self.table = (ctypes.c_void_p * len(ptrs))(*ptrs)
        self.nbytes = tensor.numel()

    def sub(self, offset: int, nbytes: int) -> "SharedBuffer":
        assert offset % 16 == 0 and offset + nbytes <= self.nbytes
        return SharedBuffer(self.tensor[offset:offset + nbytes], [p + offset for p in self.ptrs])


class _Arena:
    def __init__(self, buf: SharedBuffer):
        self.buf, self.used = buf, 0


class _EventHandle:
    """wait() makes the current stream wait for work recorded on another stream."""
    needs_sm_margin = True      # the copy runs on SMs of its own, which the GEMM beside it must leave free

    def __init__(self, event, keep=(), captured=False):
        self.event, self.keep, self.captured, self.done = event, keep, captured, False

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)
        self.done = True
        self.keep = ()


class PeerGroup:
    MAX_RANKS = _lib.MT_MAX_PEERS

    def __init__(self, group, device: torch.device):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert 1 < self.world <= self.MAX_RANKS, "peer exchange serves 2 to 8 ranks of one node"
        self.device = torch.device(device)
        self._arenas: List[_Arena] = []
        self._named: Dict[str, SharedBuffer] = {}
        self._parity: Dict[str, int] = {}
        self._imported: Dict[bytes, int] = {}
        self._side_handles: List[_EventHandle] = []
        self.side_stream = torch.cuda.Stream(device=self.device)
        self.ctrl = self.buffer("__ctrl__", _lib.MT_PEER_CTRL_BYTES)
        self.ctrl.tensor.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group)    # nobody signals a control block that its owner has not zeroed yet

    # ---- shared memory ----
    def _new_arena(self, nbytes: int) -> _Arena:
        nbytes = max(_ARENA_MIN_BYTES, (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN)
        t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        handle = (ctypes.c_uint8 * _lib.MT_IPC_HANDLE_BYTES)()
        off = ctypes.c_int64(0)
        try:
            _lib.call("mt_ipc_export", t.data_ptr(), handle, ctypes.byref(off))
            mine = (bytes(handle), int(off.value), self.device.index)
        except _lib.MtError as e:      # e.g. an allocator mode whose memory cannot be exported
            mine = (None, str(e), self.device.index)
        everyone: List[Optional[Tuple[bytes, int, int]]] = [None] * self.world
        dist.all_gather_object(everyone, mine, group=self.group)
        failed = [(r, e[1]) for r, e in enumerate(everyone) if e[0] is None]
        if failed:
            raise _lib.MtError(f"peer memory cannot be shared (rank {failed[0][0]}: {failed[0][1]})")
        ptrs = []
        for r, (h, o, _dev) in enumerate(everyone):
            if r == self.rank:
                ptrs.append(t.data_ptr())
                continue
            base = self._imported.get(h)
            if base is None:
                out = ctypes.c_void_p()
                _lib.call("mt_ipc_import", (ctypes.c_uint8 * len(h)).from_buffer_copy(h), 0, ctypes.byref(out))
                base = self._imported[h] = int(out.value)
            ptrs.append(base + o)
        arena = _Arena(SharedBuffer(t, ptrs))
        self._arenas.append(arena)
        return arena

    def buffer(self, name: str, nbytes: int) -> SharedBuffer:
        """The shared range registered under `name` (at least nbytes long); the first request on
        every rank must come in the same order, since a new arena is a collective."""
        hit = self._named.get(name)
        if hit is not None and hit.nbytes >= nbytes:
            return hit
        need = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        arena = next((a for a in self._arenas if a.buf.nbytes - a.used >= need), None)
        if arena is None:
            arena = self._new_arena(need)
        buf = arena.buf.sub(arena.used, need)
        arena.used += need
        self._named[name] = buf
        return buf

    def alternating(self, name: str, nbytes: int) -> SharedBuffer:
        """Two ranges used in turn: a range is rewritten only after a later exchange on the same
        name has passed its barrier, by which time every rank has finished reading it. Under
        stream capture the turn cannot advance from replay to replay: the first range is used
        and a barrier is issued first, which shows that every rank is done with its last use."""
        if torch.cuda.is_current_stream_capturing():
            # this rank's own pulls on the side stream count as "done" only once they have joined:
            # the barrier tells the peers that their slots may be rewritten
            for h in self._side_handles:
                if h.captured and not h.done:
                    h.wait()
            self._side_handles = [h for h in self._side_handles if not h.done]
            self.barrier()
            return self.buffer(f"{name}#0", nbytes)
        p = self._parity.get(name, 0)
        self._parity[name] = p ^ 1
        return self.buffer(f"{name}#{p}", nbytes)

    # ---- exchanges (all stream-ordered on the current stream) ----
    @staticmethod
    def _stream():
        return torch.cuda.current_stream().cuda_stream

    def barrier(self, channel: int = 0) -> None:
        _lib.call("mt_peer_barrier", self.ctrl.table, self.world, self.rank, channel, self._stream())
        kernels._count(1)

    def allreduce_max_(self, vals: torch.Tensor, channel: int = 0) -> torch.Tensor:
        """In-place MAX over the ranks of up to 4 non-negative fp32 device values; also a barrier."""
        assert vals.dtype == torch.float32 and vals.is_cuda and vals.is_contiguous() and 1 <= vals.numel() <= 4
        _lib.call("mt_peer_allreduce_max", self.ctrl.table, self.world, self.rank, channel, vals.data_ptr(), vals.numel(),
                  self._stream())
        kernels._count(1)
        return vals

    def gather(self, shared: SharedBuffer, segments, ctas: int = 296, whole_sms: bool = False) -> None:
        """segments: (byte offset inside every rank's shared range, destination tensor, shard bytes).
        whole_sms: `ctas` CTAs that each take one SM, for a copy that runs beside a GEMM which leaves
        that many SMs free."""
        n = len(segments)
        offs = (ctypes.c_int64 * n)(*[s[0] for s in segments])
        dsts = (ctypes.c_void_p * n)(*[s[1].data_ptr() for s in segments])
        sizes = (ctypes.c_int64 * n)(*[s[2] for s in segments])
        _lib.call("mt_peer_gather", shared.table, self.world, self.rank, offs, dsts, sizes, n, ctas, int(whole_sms), self._stream())
        kernels._count(1)

    def reduce_bf16(self, stage: SharedBuffer, rows: int, cols: int, amax_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=self.device)
        _lib.call("mt_peer_reduce_bf16", stage.tensor.data_ptr(), self.world, rows, cols, out.data_ptr(),
                  None if amax_out is None else amax_out.data_ptr(), self._stream())
        kernels._count(1)
        return out

    def on_side_stream(self, fn, keep=()) -> _EventHandle:
        """Runs fn() on the side stream, ordered after the work already enqueued on the current
        stream; the returned handle's wait() orders later work of the current stream after it."""
        main = torch.cuda.current_stream()
        capturing = torch.cuda.is_current_stream_capturing()
        self.side_stream.wait_stream(main)
        with torch.cuda.stream(self.side_stream):
            fn()
            ev = torch.cuda.Event()
            ev.record(self.side_stream)
        h = _EventHandle(ev, keep, captured=capturing)
        if capturing:
            self._side_handles.append(h)
        return h


_GROUPS: Dict[int, Optional[PeerGroup]] = {}


def get_peer_group(group, device) -> Optional[PeerGroup]:
    """The PeerGroup of a process group (created on first use, a collective), or None when the
    group is not a set of 2..8 CUDA ranks whose memory can be shared (callers then keep to NCCL)."""
    if group is None or not dist.is_initialized():
        return None
    key = id(group)
    if key not in _GROUPS:
        pg = None
        world = dist.get_world_size(group)
        ok = 1 < world <= PeerGroup.MAX_RANKS and torch.device(device).type == "cuda" and dist.get_backend(group) == "nccl"
        # every rank must agree before the collectives inside PeerGroup() start
        flag = torch.tensor([1 if ok else 0], device=device if ok else "cpu")
        if ok:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            if int(flag.item()) == 1:
                try:
                    pg = PeerGroup(group, device)
                except _lib.MtError as e:       # raised on every rank together (see _new_arena)
                    import warnings
                    warnings.warn(f"peer-memory exchange unavailable, keeping to the process group: {e}")
                    pg = None
        _GROUPS[key] = pg
    return _GROUPS[key]
