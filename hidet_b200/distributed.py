"""Column-parallel quantized linear over the GPUs of one node.

The reference has no sharding layer: the user slices weights by hand and inserts collectives
(examples/distributed/test.py); its collective op is an NCCL all-gather whose result is rank-major,
``[nranks, *x.shape]`` (python/hidet/graph/ops/distributed.py:63-97).  This module provides that
op with the same result layout, and on top of it the one strategy this path needs: split the weight
along N, one process per GPU, gather the output slices.

Per-output-channel quantization is column-local, so quantizing a column shard gives exactly the
columns of the quantized full weight; a rank only ever needs its own shard.

torch.distributed is the plumbing (NCCL on GPUs; the host logic also runs under gloo on CPU, where
only the gathering can be exercised because the kernels are CUDA-only).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def column_range(n: int, rank: int, world: int, multiple: int = 16) -> Tuple[int, int]:
    """Columns [begin, end) of rank `rank`.  N must split into equal blocks that are multiples of
    `multiple` columns (16 keeps every shard's rows 16-byte multiples for the TMA kernels)."""
    if n % (world * multiple) != 0:
        raise ValueError('N={} does not split into {} equal column blocks of a multiple of {}'.format(n, world, multiple))
    step = n // world
    return rank * step, (rank + 1) * step


def shard_columns(weight: torch.Tensor, scale: Optional[torch.Tensor], rank: int, world: int):
    """The contiguous column shard of a [K, N] weight (quantized or not) and of its [N] scale."""
    begin, end = column_range(weight.shape[-1], rank, world)
    w = weight[..., begin:end].contiguous()
    s = scale[begin:end].contiguous() if scale is not None else None
    return w, s


def all_gather(x: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rank-major gather, the reference op's contract: returns y[nranks, *x.shape] with y[r] = x of rank r."""
    world = dist.get_world_size(group)
    x = x.contiguous()
    if out is None:
        out = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out.view(-1), x.view(-1), group=group)
    return out


def gather_columns(c_local: torch.Tensor, group=None, out: Optional[torch.Tensor] = None,
                   staging: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Output slices c_local[..., M, N/g] of all ranks -> c[..., M, N] on every rank.

    The all-gather delivers [g, M, N/g]; for a single row that already is [M, N]; otherwise one
    strided copy puts the slices side by side."""
    world = dist.get_world_size(group)
    lead = tuple(c_local.shape[:-1])
    n_local = c_local.shape[-1]
    rows = 1
    for d in lead:
        rows *= d
    gathered = all_gather(c_local.reshape(rows, n_local), group=group, out=staging)  # [g, rows, n_local]
    if out is None:
        out = torch.empty(lead + (world * n_local,), dtype=c_local.dtype, device=c_local.device)
    if rows == 1:
        out.view(-1).copy_(gathered.view(-1))
    else:
        out.view(rows, world, n_local).copy_(gathered.permute(1, 0, 2))
    return out


class PeerOutput:
    """A [rows, cols] float16 output buffer that exists on every rank of the group and that every
    rank can store into directly: symmetric memory (torch.distributed._symmetric_memory), i.e. the
    same allocation on every GPU, peer-mapped over NVLink.  Two copies are kept and used in turn, so
    that a rank may still read the previous result while its peers already write the next one.
    """

    def __init__(self, rows: int, cols: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.buffers, self.handles, self.ptr_tables, self.multicast_ptrs = [], [], [], []
        for _ in range(2):
            buf = symm_mem.empty((rows, cols), dtype=torch.float16, device=device)
            handle = symm_mem.rendezvous(buf, group)
            self.buffers.append(buf)
            self.handles.append(handle)
            self.ptr_tables.append([int(p) for p in handle.buffer_ptrs])
            # non-zero when the allocation is also bound to an NVLink multicast object (NVSwitch systems)
            self.multicast_ptrs.append(int(getattr(handle, 'multicast_ptr', 0) or 0))
        self.turn = 0

    def release(self) -> None:
        """Drops the buffers, handles and pointer tables.  Call it on every rank before the process group is
        destroyed (and before a rank exits), while no kernel that stores to a peer is in flight: memory that
        is still peer-mapped when its owner goes away faults the GPUs that map it."""
        self.buffers, self.handles, self.ptr_tables, self.multicast_ptrs = [], [], [], []

    def next(self):
        """(local buffer, table of every rank's pointer to its copy, handle, multicast pointer or 0) for the next result."""
        i = self.turn
        self.turn ^= 1
        return self.buffers[i], self.ptr_tables[i], self.handles[i], self.multicast_ptrs[i]


class ColumnParallelQuantLinear:
    """y = x @ dequant(Wq, scale) with Wq[K, N] split along N over the ranks of `group`.

    Build it from this rank's shard of the unquantized weight (`from_weight_shard`) or from an
    already quantized shard.  `forward` runs the local quantized matmul and delivers the slices:

    gather='nccl'  the local kernel writes its slice, an NCCL all-gather collects the slices
                   (rank-major, as the reference's all-gather op) and one copy puts them side by side;
    gather='p2p'   every rank's [M, N] output is peer-mapped on all ranks (symmetric memory), and the kernel's
                   epilogue stores its columns straight into every rank's output over NVLink, tile by tile
                   while the rest of the product is still being computed (b200q_qlinear_f16_i8_to_peers); where the
                   outputs are also bound to an NVLink multicast object, large M stores once to the multicast
                   address and the switch delivers to all ranks (b200q_qlinear_f16_i8_to_multicast).
                   One cross-rank barrier on the stream follows: no staging buffer, no reshuffle, no
                   collective launch.
    """

    MULTICAST_MIN_ROWS = 33   # what the large-M kernel serves
    MULTICAST_MIN_WORLD = 4   # with one peer a multicast store only adds this GPU's own copy to the link traffic (measured: slower)

    def __init__(self, wq_shard: torch.Tensor, scale_shard: torch.Tensor, group=None, gather: str = 'nccl', multicast: bool = True):
        if wq_shard.dtype != torch.int8 or wq_shard.dim() != 2:
            raise ValueError('expect an int8 [K, N/g] weight shard')
        if gather not in ('nccl', 'p2p'):
            raise ValueError("gather must be 'nccl' or 'p2p', got {!r}".format(gather))
        self.wq = wq_shard.contiguous()
        self.scale = scale_shard.contiguous()
        self.group = group
        self.gather = gather
        self.multicast = multicast   # use the NVLink multicast mapping of the outputs for large M where there is one
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if gather == 'p2p' and self.world > 8:
            raise ValueError('peer stores serve up to 8 ranks, got {}'.format(self.world))
        self._buffers = {}
        self._peer_outputs = {}

    @classmethod
    def from_weight_shard(cls, w_shard: torch.Tensor, group=None, gather: str = 'nccl', multicast: bool = True):
        from .quant import symmetric_quantize

        wq, scale = symmetric_quantize(w_shard, 'int8', dims=0)
        return cls(wq, scale, group, gather, multicast)

    def share_outputs_with(self, other: 'ColumnParallelQuantLinear') -> None:
        """Use `other`'s peer-mapped output buffers (layers of equal width that run one after the
        other can share them; every layer that owns its own costs two [M, N] buffers per shape)."""
        self._peer_outputs = other._peer_outputs

    def release(self) -> None:
        """Gives up the peer-mapped outputs and gather buffers (see PeerOutput.release)."""
        for peer_out in self._peer_outputs.values():
            peer_out.release()
        self._peer_outputs = {}
        self._buffers = {}

    @property
    def in_features(self) -> int:
        return self.wq.shape[0]

    @property
    def out_features(self) -> int:
        return self.wq.shape[1] * self.world

    def local(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        from .quant import symmetric_quant_matmul

        return symmetric_quant_matmul(x, self.wq, self.scale, out=out)

    def _forward_p2p(self, x: torch.Tensor) -> torch.Tensor:
        import ctypes

        from . import ffi
        from .runtime import workspaces

        lead = tuple(x.shape[:-1])
        rows = 1
        for d in lead:
            rows *= d
        k, n_local = self.wq.shape
        n = n_local * self.world
        key = (rows, x.device)
        if key not in self._peer_outputs:
            self._peer_outputs[key] = PeerOutput(rows, n, x.device, self.group)
        out, ptrs, handle, multicast_ptr = self._peer_outputs[key].next()
        x = x.contiguous()
        c0 = self.rank * n_local
        qlinear = ffi.func('b200q_qlinear_f16_i8_to_peers')
        with torch.cuda.device(x.device):
            ws_bytes = ffi.func('b200q_qlinear_workspace_bytes')(rows, n_local, k, ffi.LAYOUT_KN)
            ws_ptr, ws_size = workspaces.get(x.device, ws_bytes)
            main = torch.cuda.current_stream(x.device)
            if multicast_ptr and self.multicast and rows >= self.MULTICAST_MIN_ROWS and self.world >= self.MULTICAST_MIN_WORLD:
                # large M: every 16 bytes leave this GPU once and the switch delivers them to all ranks
                ffi.func('b200q_qlinear_f16_i8_to_multicast')(x.data_ptr(), self.wq.data_ptr(), self.scale.data_ptr(), multicast_ptr, n, c0,
                                                            rows, n_local, k, ws_ptr, ws_size, main.cuda_stream)
            else:
                table = (ctypes.c_void_p * self.world)(*ptrs)
                qlinear(x.data_ptr(), self.wq.data_ptr(), self.scale.data_ptr(), table, self.world, n, c0, rows, n_local, k,
                        ws_ptr, ws_size, main.cuda_stream)
            handle.barrier(channel=0)  # on the current stream: every rank's columns have landed everywhere
        return out.view(lead + (n,))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.gather == 'p2p':
            return self._forward_p2p(x)
        lead = tuple(x.shape[:-1])
        key = (lead, x.device)
        if key not in self._buffers:  # static buffers: a decode loop calls this with the same shape every step
            rows = 1
            for d in lead:
                rows *= d
            n_local = self.wq.shape[1]
            self._buffers[key] = (
                torch.empty(lead + (n_local,), dtype=torch.float16, device=x.device),
                torch.empty((self.world, rows, n_local), dtype=torch.float16, device=x.device),
                torch.empty(lead + (self.out_features,), dtype=torch.float16, device=x.device),
            )
        c_local, staging, out = self._buffers[key]
        self.local(x, out=c_local)
        return gather_columns(c_local, self.group, out=out, staging=staging)

    __call__ = forward
