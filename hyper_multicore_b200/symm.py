"""Peer-mapped workspace for expert parallelism: one cudaMalloc per rank, CUDA-IPC handles
exchanged once through torch.distributed, raw peer pointers handed to the kernels.

This is the CUDA counterpart of the reference's symmetric heap for the MoE path
(hyper_multicore/shmem/_api.py:77-182, hyper_multicore/modules/mega_moe/workspace.py:48-75,
409-470): a receive buffer for dispatched rows, a routed buffer for returning rows, and a control
block with per-expert arrival counters, the combine counter and persistent ready flags.
NCCL / Gloo is used only for the handle exchange.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from . import _lib

_ALIGN_ROWS = 128


def align_rows(rows: int) -> int:
    """Round a row capacity up to the 128-row communication split the reference uses."""
    return max(_ALIGN_ROWS, (rows + _ALIGN_ROWS - 1) // _ALIGN_ROWS * _ALIGN_ROWS)


class _DeviceSpan:
    """Expose raw device memory to torch through __cuda_array_interface__ (no copy)."""

    def __init__(self, address: int, nbytes: int, owner: Any) -> None:
        self.owner = owner
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 3, "strides": None,
        }


def _map_peers(lib, base: ctypes.c_void_p, nbytes: int, group: Any, ep: int, rank: int):
    """Exchange CUDA-IPC handles of one allocation; returns (addresses of every rank's copy, opened)."""
    if ep == 1:
        return [base.value], []
    handle = (ctypes.c_ubyte * 64)()
    _lib.check(lib.hmc_ipc_get_handle(base, handle))
    gathered: list[Any] = [None] * ep
    dist.all_gather_object(gathered, (bytes(handle), nbytes), group=group)
    bases, opened = [], []
    for peer, (peer_handle, peer_bytes) in enumerate(gathered):
        if peer_bytes != nbytes:
            raise RuntimeError("EP ranks disagree on the size of a peer-mapped allocation")
        if peer == rank:
            bases.append(base.value)
            continue
        mapped = ctypes.c_void_p()
        raw = (ctypes.c_ubyte * 64).from_buffer_copy(peer_handle)
        _lib.check(lib.hmc_ipc_open_handle(raw, ctypes.byref(mapped)))
        bases.append(mapped.value)
        opened.append(mapped.value)
    dist.barrier(group=group)  # every rank has mapped every peer before anyone may write remotely
    return bases, opened


class PeerControl:
    """The part of the peer-mapped state that outlives workspace growth: the control block and the
    table of the count exchange. Created collectively at the first call of an EP group member
    (the reference keeps its signal arena and route header in the symmetric heap the same way,
    hyper_multicore/modules/mega_moe/workspace.py:409-470)."""

    def __init__(self, group: Any, experts: int, device: torch.device) -> None:
        self.group, self.device, self.experts = group, device, experts
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.ep > _lib.HMC_MAX_EP:
            raise ValueError(f"expert-parallel size {self.ep} exceeds the supported maximum {_lib.HMC_MAX_EP}")
        lib = _lib.load()
        self._ctrl_bytes = _lib.HMC_CTRL_WORDS * 4
        self._table_off = (self._ctrl_bytes + 1023) // 1024 * 1024
        self._table_bytes = int(lib.hmc_ep_exchange_table_bytes(self.ep, experts))
        self.nbytes = self._table_off + self._table_bytes
        self._base = ctypes.c_void_p()
        self._closed = False
        self.generation = 0   # operator calls (dispatch / combine phases)
        self.exchanges = 0    # count exchanges
        with torch.cuda.device(device):
            _lib.check(lib.hmc_symm_alloc(self.nbytes, ctypes.byref(self._base)))
            self._peer_bases, self._opened = _map_peers(lib, self._base, self.nbytes, group, self.ep, self.rank)
        span = torch.as_tensor(_DeviceSpan(self._base.value, self.nbytes, self), device=device)
        self.ctrl = span[:self._ctrl_bytes].view(torch.int32)
        self.table = span[self._table_off:self.nbytes].view(torch.int32).view(2, self.ep * (experts + 4))
        # the route guard's decision, one word per exchange parity: a call's kernels may still read theirs
        # while the next call's guard writes the other
        self._skip_flags = torch.zeros(2, dtype=torch.int32, device=device)
        pointer_array = ctypes.c_void_p * self.ep
        self.peer_ctrl = pointer_array(*self._peer_bases)
        self.peer_tables = pointer_array(*(base + self._table_off for base in self._peer_bases))

    def exchange(self, counts: torch.Tensor, header: tuple[int, int, int], status, budget_ns: int):
        """Returns (counts [ep, experts], raw block [ep * (experts + 4)]) of this exchange, on the device."""
        from . import kernels  # pylint: disable=import-outside-toplevel

        self.exchanges += 1
        args = _lib.EpExchangeArgs()
        args.counts = counts.data_ptr()
        args.header[0], args.header[1], args.header[2], args.header[3] = header[0], header[1], header[2], 0
        args.peer_tables = ctypes.cast(self.peer_tables, ctypes.c_void_p)
        args.peer_ctrl = ctypes.cast(self.peer_ctrl, ctypes.c_void_p)
        args.local_ctrl = self.ctrl.data_ptr()
        args.ep, args.rank, args.experts = self.ep, self.rank, self.experts
        args.exchange, args.budget_ns = self.exchanges, budget_ns
        args.status = _lib.ptr(status)
        kernels._call("hmc_ep_exchange_counts", self.device, ctypes.byref(args))  # pylint: disable=protected-access
        block = self.table[self.exchanges & 1]
        return block[:self.ep * self.experts].view(self.ep, self.experts), block

    @property
    def skip_flag(self) -> torch.Tensor:
        """Device word of the current exchange that the operator's kernels consult."""
        return self._skip_flags[self.exchanges & 1:(self.exchanges & 1) + 1]

    def close(self) -> None:
        """Collective: unmap peers and free."""
        if self._closed:
            return
        self._closed = True
        lib = _lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            if dist.is_initialized():
                dist.barrier(group=self.group)
            for mapped in self._opened:
                lib.hmc_ipc_close_handle(ctypes.c_void_p(mapped))
            if dist.is_initialized():
                dist.barrier(group=self.group)
            lib.hmc_symm_free(self._base)
        self._opened = []


class PeerWorkspace:
    """Symmetric allocation of one EP group member, with every peer's copy mapped locally."""

    def __init__(self, group: Any | None, hidden_size: int, capacity_rows: int, routed_rows: int,
                 device: torch.device, pull: bool = False, control: "PeerControl | None" = None) -> None:
        """``pull``: the first buffer is this rank's SOURCE buffer (its own rows in expert-major order,
        read by the owners), so it holds ``routed_rows`` rows and no receive capacity is needed."""
        self.group = group
        self.device = device
        self.hidden_size = hidden_size
        self.ep = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if self.ep > _lib.HMC_MAX_EP:
            raise ValueError(f"expert-parallel size {self.ep} exceeds the supported maximum {_lib.HMC_MAX_EP}")
        self.pull = pull
        self.routed_rows = align_rows(routed_rows)
        self.capacity_rows = self.routed_rows if pull else align_rows(capacity_rows)
        self.generation = 0
        self._base = ctypes.c_void_p()
        self._peer_bases: list[int] = []
        self._opened: list[int] = []
        self._closed = False
        row_bytes = hidden_size * 2
        self._ctrl_bytes = _lib.HMC_CTRL_WORDS * 4
        self._expert_off = (self._ctrl_bytes + 1023) // 1024 * 1024
        # One float per row follows each buffer (routing probabilities travelling with dispatched rows,
        # probability gradients travelling back with combined rows).
        self.expert_plane_offset = self.capacity_rows * row_bytes
        self.routed_plane_offset = self.routed_rows * row_bytes
        self._routed_off = self._expert_off + self.expert_plane_offset + self.capacity_rows * 4
        self.nbytes = self._routed_off + self.routed_plane_offset + self.routed_rows * 4
        lib = _lib.load()
        with torch.cuda.device(device):
            _lib.check(lib.hmc_symm_alloc(self.nbytes, ctypes.byref(self._base)))
            self._exchange_handles(lib)
        span = torch.as_tensor(_DeviceSpan(self._base.value, self.nbytes, self), device=device)
        self._bytes = span
        self.ctrl = span[:self._ctrl_bytes].view(torch.int32)
        expert_end = self._expert_off + self.expert_plane_offset
        routed_end = self._routed_off + self.routed_plane_offset
        self.expert_buffer = span[self._expert_off:expert_end].view(torch.bfloat16).view(
            self.capacity_rows, hidden_size)
        self.expert_values = span[expert_end:self._routed_off].view(torch.float32)
        self.routed_buffer = span[self._routed_off:routed_end].view(torch.bfloat16).view(
            self.routed_rows, hidden_size)
        self.routed_values = span[routed_end:self.nbytes].view(torch.float32)
        # pull mode reads the same memory under the names of its role
        self.source_buffer, self.source_values = self.expert_buffer, self.expert_values
        self.source_plane_offset = self.expert_plane_offset
        pointer_array = ctypes.c_void_p * self.ep
        self.peer_ctrl = pointer_array(*self._peer_bases)
        self.control = control
        if control is not None:
            # the control block (and the generation counter) outlive this buffer allocation
            self.ctrl, self.peer_ctrl = control.ctrl, control.peer_ctrl
        self.peer_expert = pointer_array(*(base + self._expert_off for base in self._peer_bases))
        self.peer_routed = pointer_array(*(base + self._routed_off for base in self._peer_bases))
        self.peer_source = self.peer_expert

    def _exchange_handles(self, lib: ctypes.CDLL) -> None:
        if self.ep == 1:
            self._peer_bases = [self._base.value]
            return
        handle = (ctypes.c_ubyte * 64)()
        _lib.check(lib.hmc_ipc_get_handle(self._base, handle))
        gathered: list[Any] = [None] * self.ep
        dist.all_gather_object(gathered, (bytes(handle), self.nbytes), group=self.group)
        for peer, (peer_handle, peer_bytes) in enumerate(gathered):
            if peer_bytes != self.nbytes:
                raise RuntimeError("EP ranks disagree on the symmetric workspace size")
            if peer == self.rank:
                self._peer_bases.append(self._base.value)
                continue
            mapped = ctypes.c_void_p()
            raw = (ctypes.c_ubyte * 64).from_buffer_copy(peer_handle)
            _lib.check(lib.hmc_ipc_open_handle(raw, ctypes.byref(mapped)))
            self._peer_bases.append(mapped.value)
            self._opened.append(mapped.value)
        # every rank has mapped every peer before anyone may write remotely
        dist.barrier(group=self.group)

    def next_generation(self) -> int:
        """Generation number of the next operator call (same sequence on every rank)."""
        if self.control is not None:
            self.control.generation += 1
            self.generation = self.control.generation
            return self.generation
        self.generation += 1
        return self.generation

    def begin_call(self) -> int:
        """Zero the per-call counters on the current stream, then tell every peer this rank's
        buffers are free for the new generation. Returns the generation."""
        generation = self.next_generation()
        self.ctrl[:_lib.HMC_CTRL_READY].zero_()
        from . import kernels  # pylint: disable=import-outside-toplevel

        kernels._call("hmc_ep_publish_ready", self.device, self.peer_ctrl, self.ep, self.rank, generation)  # pylint: disable=protected-access
        return generation

    def debug_state(self) -> dict:
        """Sizes, peer map and the current control words (synchronises the device)."""
        words = self.ctrl.tolist()
        return {
            "ep": self.ep, "rank": self.rank, "bytes": self.nbytes, "capacity_rows": self.capacity_rows,
            "routed_rows": self.routed_rows, "generation": self.generation,
            "peer_bases": [hex(p) for p in self._peer_bases],
            "combine_counter": words[_lib.HMC_CTRL_COMBINE],
            "ready": [words[_lib.HMC_CTRL_READY + p * _lib.HMC_CTRL_READY_STRIDE] for p in range(self.ep)],
        }

    def close(self) -> None:
        """Unmap peers and free the local allocation. Collective for ep > 1."""
        if self._closed:
            return
        self._closed = True
        lib = _lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            if self.ep > 1 and dist.is_initialized():
                dist.barrier(group=self.group)  # no peer may still be writing into this rank
            for mapped in self._opened:
                lib.hmc_ipc_close_handle(ctypes.c_void_p(mapped))
            if self.ep > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            lib.hmc_symm_free(self._base)
        self._opened = []

    def __del__(self) -> None:
        # Collective teardown cannot run from a finaliser; only a single-rank workspace frees itself.
        if not self._closed and self.ep == 1:
            try:
                self.close()
            except Exception:  # pylint: disable=broad-except
                pass
