"""Multi-GPU forms of the operator (one process per GPU, ``torch.distributed``).

The reference is single-GPU.  Two partitionings follow from the structure of
the algorithm:

* **Rows** are independent, so a batch is sharded row-wise and every rank runs
  the plain operator on its rows.  No collective is involved
  (:func:`row_shard`, :func:`topk_row_sharded`).

* **One very long row** with interleaved buckets is a ``stripes x b`` matrix;
  rank ``g`` of ``G`` owns the contiguous *bucket group* (columns)
  ``[g*b/G, (g+1)*b/G)`` as a dense ``stripes x b/G`` slab in its own memory.
  Stage 1 is independent per bucket, so each rank produces exactly the slice
  ``[g*k0/G, (g+1)*k0/G)`` of the single-GPU candidate buffer (slot =
  ``bucket*j + q``).  One all-gather of the (value, index) candidates over
  NVLink reassembles that buffer on every rank, and the exact select over it
  gives the same answer as one GPU would (:func:`topk_long_row`).

The candidates land in each GPU's own memory before the select reads them, either
by the collective or, with ``exchange="push"`` (:class:`LongRowTopK`), by one kernel
per rank that stores the rank's block into the peers' buffers over NVLink; no kernel
loads from a peer's memory and none waits for another GPU.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist
from torch import Tensor

from . import _native


def row_shard(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open row range of ``rank`` when ``rows`` rows are split as evenly as
    possible over ``world`` ranks (the first ``rows % world`` ranks get one more)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def topk_row_sharded(xs_local: Tensor, k: int, j: int = 1, k_mult: int = 1,
                     interleaved: bool = True) -> tuple[Tensor, Tensor]:
    """The operator on this rank's rows.  Exists for symmetry with
    :func:`topk_long_row`; it is the plain operator because rows never interact."""
    from .priority_queue import topk

    return topk(xs_local, k, -1, j=j, k_mult=k_mult, interleaved=interleaved)


def bucket_group(total_buckets: int, rank: int, world: int) -> tuple[int, int]:
    """Columns ``[start, stop)`` of the ``stripes x total_buckets`` view owned by ``rank``.

    Every rank gets ``ceil(total_buckets / world)`` columns until the columns run
    out, so when the world size does not divide the bucket count the last groups
    are short (possibly empty).  All real columns therefore precede all padding,
    and after an all-gather of equal-sized candidate blocks the first ``k0`` slots
    of the gathered buffer are exactly the single-GPU candidate buffer."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    cols = group_width(total_buckets, world)
    return min(total_buckets, rank * cols), min(total_buckets, (rank + 1) * cols)


def group_width(total_buckets: int, world: int) -> int:
    """Columns of a full bucket group: ``ceil(total_buckets / world)``."""
    return -(-total_buckets // world)


def slab_of_row(row: Tensor, total_buckets: int, rank: int, world: int) -> Tensor:
    """Cut this rank's dense ``stripes x cols`` slab out of a full row (used by
    tests and single-node drivers that start from the whole row)."""
    n = row.numel()
    if n % total_buckets:
        raise ValueError("the row length must be a multiple of the number of buckets")
    start, stop = bucket_group(total_buckets, rank, world)
    return row.view(n // total_buckets, total_buckets)[:, start:stop].contiguous()


def _native_stage1_slab(slab: Tensor, total_buckets: int, col_offset: int, j: int,
                        out: tuple[Tensor, Tensor] | None = None,
                        workspace: Tensor | None = None) -> tuple[Tensor, Tensor]:
    _native.require_cuda(slab)
    _native.require_device(slab.device)
    # the kernel reads a dense stripes x cols array: a strided view (a column
    # range cut out of the full row) is copied, never read through its base pointer
    slab = slab.contiguous()
    stripes, cols = slab.shape
    if out is None:
        vals = torch.empty(cols * j, device=slab.device, dtype=slab.dtype)
        idx = torch.empty(cols * j, device=slab.device, dtype=torch.int64)
    else:
        vals, idx = out
    lib = _native.lib()
    code = _native.dtype_code(slab.dtype)
    with torch.cuda.device(slab.device):
        if workspace is None:
            ws_bytes = lib.atk_stage1_slab_workspace_bytes(code, stripes, cols, j)
            workspace = torch.empty(ws_bytes, device=slab.device, dtype=torch.uint8) if ws_bytes else None
        ws_bytes = workspace.numel() if workspace is not None else 0
        status = lib.atk_stage1_slab(
            slab.data_ptr(), code, stripes, cols, total_buckets, col_offset, j,
            vals.data_ptr(), idx.data_ptr(), workspace.data_ptr() if ws_bytes else None, ws_bytes,
            _native.current_stream_ptr(slab.device))
    _native.check(status)
    return vals, idx


def _native_select(cand_vals: Tensor, cand_idx: Tensor, k: int,
                   out: tuple[Tensor, Tensor] | None = None,
                   workspace: Tensor | None = None) -> tuple[Tensor, Tensor]:
    _native.require_cuda(cand_vals)
    k0 = cand_vals.numel()
    code = _native.dtype_code(cand_vals.dtype)
    lib = _native.lib()
    if out is None:
        vals = torch.empty(k, device=cand_vals.device, dtype=cand_vals.dtype)
        idx = torch.empty(k, device=cand_vals.device, dtype=torch.int64)
    else:
        vals, idx = out
    with torch.cuda.device(cand_vals.device):
        if workspace is None:
            ws_bytes = lib.atk_select_workspace_bytes(code, 1, k0, k)
            workspace = torch.empty(ws_bytes, device=cand_vals.device, dtype=torch.uint8) if ws_bytes else None
        ws_bytes = workspace.numel() if workspace is not None else 0
        status = lib.atk_select(cand_vals.data_ptr(), cand_idx.data_ptr(), code, 1, k0, k0, k,
                                vals.data_ptr(), idx.data_ptr(), k,
                                workspace.data_ptr() if ws_bytes else None, ws_bytes,
                                _native.current_stream_ptr(cand_vals.device))
    _native.check(status)
    return vals, idx


class _RawCudaBytes:
    """Lets torch view device memory it did not allocate (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerBuffers:
    """One buffer of ``nbytes`` bytes per rank of a node, each mapped into every rank.

    ``local`` is this rank's buffer as a ``uint8`` tensor (zero-filled); ``ptrs[r]`` is the
    address of rank ``r``'s buffer in THIS process, valid in kernels of this rank's GPU
    (CUDA interprocess handles, opened with this rank's device current; peer access is
    enabled by the mapping).  The handles travel over the process group.  Set-up and
    :meth:`close` are collective and synchronise; neither may run inside a graph capture.
    """

    def __init__(self, nbytes: int, device: torch.device, group: dist.ProcessGroup | None = None):
        import ctypes

        self.group, self.device, self.nbytes = group, torch.device(device), nbytes
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        lib = _native.lib()
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        self._own, self.local = None, None
        self.ptrs: list[int] = []
        self._opened: list[int] = []
        # A failure on any rank (no memory, a peer's GPU hidden from a process, no peer access)
        # becomes the same RuntimeError on EVERY rank, after everything has been released: the
        # ranks agree on the outcome of each step before the next.
        problem = None
        with torch.cuda.device(self.device):
            status = lib.atk_peer_alloc(nbytes, ctypes.byref(own), handle)
        if status != _native.ATK_OK:
            problem = f"cannot allocate {nbytes} bytes: {_native.strerror(status)}"
        else:
            self._own = own.value
        handles: list = [None] * self.world
        dist.all_gather_object(handles, (problem, self.device.index, bytes(handle.raw)), group=group)
        self._raise_together([h[0] for h in handles])
        with torch.cuda.device(self.device):
            for r, (_, peer_device, raw) in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self._own)
                    continue
                mapped = ctypes.c_void_p()
                if peer_device == self.device.index:
                    problem = f"rank {r} uses the same device index {peer_device}: the GPUs of all ranks must be visible to every rank"
                elif not torch.cuda.can_device_access_peer(self.device.index, peer_device):
                    problem = f"GPU {self.device.index} has no peer access to GPU {peer_device} (rank {r})"
                else:
                    status = lib.atk_peer_open(ctypes.create_string_buffer(raw, 64), ctypes.byref(mapped))
                    if status != _native.ATK_OK:
                        problem = f"cannot map the buffer of rank {r}: {_native.strerror(status)}"
                if problem is not None:
                    break
                self.ptrs.append(mapped.value)
                self._opened.append(mapped.value)
        outcomes: list = [None] * self.world
        dist.all_gather_object(outcomes, problem, group=group)
        self._raise_together(outcomes)
        self.local = torch.as_tensor(_RawCudaBytes(self._own, nbytes), device=self.device)

    def _raise_together(self, problems: list) -> None:
        """Every rank holds the same list: release and raise on all of them if any rank failed."""
        failed = [(r, p) for r, p in enumerate(problems) if p is not None]
        if not failed:
            return
        self._release()                       # every rank: it holds a barrier
        raise RuntimeError("PeerBuffers: " + "; ".join(f"rank {r}: {p}" for r, p in failed))

    def close(self) -> None:
        """Collective: every rank unmaps its peers' buffers, then the owners free them."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self._release()

    def _release(self) -> None:
        lib = _native.lib()
        with torch.cuda.device(self.device):
            for ptr in self._opened:
                lib.atk_peer_close(ptr)
            self._opened = []
            if dist.is_initialized():
                try:
                    dist.barrier(self.group)          # no owner frees while a peer still maps its buffer
                except Exception:                     # the group is already gone: nothing left to order
                    pass
            if self._own is not None:
                lib.atk_peer_free(self._own)
        self._own, self.local, self.ptrs = None, None, []


class LongRowTopK:
    """The long-row operator with every buffer allocated once.

    A step (:meth:`__call__`) launches stage 1 on this rank's slab, the all-gather
    of the candidates and the exact select, all on the current stream and without
    allocating or synchronising, so a step can be captured in a CUDA graph
    together with its NCCL collective.  Results are written to ``self.values`` /
    ``self.indices`` (overwritten by the next step).

    ``events``, when given to a step, receives one recorded CUDA event after each
    phase (stage 1, exchange, select) for a per-phase breakdown.

    ``exchange`` picks how the candidates travel:

    * ``"all_gather"`` (default): one NCCL all-gather of the packed blocks into every
      rank's own memory, then two copies that unpack them.
    * ``"push"`` (ranks of one node with peer access): every rank maps the candidate
      buffers of all ranks once (:class:`PeerBuffers`), stage 1 writes this rank's
      block into its own buffer, ONE kernel (``atk_push_blocks``) stores the block into
      every peer's buffer over NVLink, and a one-element all-reduce orders the ranks'
      streams before the select reads.  Nothing is unpacked and no rank loads from a
      peer.  The buffers exist twice and steps alternate between them, so a rank that
      runs ahead never writes into a buffer a peer is still selecting from; for the same
      reason a CUDA graph that is replayed must hold an EVEN number of steps, and eager
      steps must not be mixed in between replays of such a graph (two consecutive steps
      would then use the same buffers).  Call
      :meth:`close` (collective) when done, before the process group is destroyed.
    """

    def __init__(self, stripes: int, k: int, j: int, k_mult: int, dtype: torch.dtype,
                 device: torch.device, group: dist.ProcessGroup | None = None,
                 exchange: str = "all_gather"):
        if exchange not in ("all_gather", "push"):
            raise ValueError(f"exchange must be 'all_gather' or 'push', was {exchange!r}")
        if k_mult < 1:
            raise ValueError(f"k_mult must be >=1, was {k_mult}")
        self.k, self.j, self.k_mult = k, j, k_mult
        self.k0 = k * k_mult
        if self.k0 % j:
            raise RuntimeError("topk: j must divide k")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.total_buckets = self.k0 // j
        self.start, self.stop = bucket_group(self.total_buckets, self.rank, self.world)
        self.cols = self.stop - self.start
        self.stripes = stripes
        self.dtype, self.device = dtype, torch.device(device)
        block = group_width(self.total_buckets, self.world) * j      # candidates per rank, padded groups included
        self.block = block
        lib = _native.lib()
        code = _native.dtype_code(dtype)
        dev = self.device
        esize = torch.empty(0, dtype=dtype).element_size()
        self.exchange = exchange if self.world > 1 else "none"
        self._step = 0
        with torch.cuda.device(dev):
            if self.exchange == "push":
                self._init_push(block, esize)
            elif self.world > 1:
                # One exchange instead of two: a rank's positions and values travel in one
                # packed block [block x int64 | block x dtype, padded to 16 bytes]; stage 1
                # writes straight into views of it, and the gathered blocks are unpacked into
                # the dense candidate arrays the select reads.
                self._idx_bytes = block * 8
                self._block_bytes = (self._idx_bytes + block * esize + 15) // 16 * 16
                self._packed_local = torch.empty(self._block_bytes, device=dev, dtype=torch.uint8)
                self._packed_all = torch.empty(self._block_bytes * self.world, device=dev, dtype=torch.uint8)
                self.local_idx = self._packed_local[:self._idx_bytes].view(torch.int64)
                self.local_vals = self._packed_local[self._idx_bytes:self._idx_bytes + block * esize].view(dtype)
                self.cand_vals = torch.empty(block * self.world, device=dev, dtype=dtype)
                self.cand_idx = torch.empty(block * self.world, device=dev, dtype=torch.int64)
            else:
                self.local_vals = torch.empty(block, device=dev, dtype=dtype)
                self.local_idx = torch.empty(block, device=dev, dtype=torch.int64)
                self.cand_vals, self.cand_idx = self.local_vals, self.local_idx
            ws1 = lib.atk_stage1_slab_workspace_bytes(code, stripes, self.cols, j) if self.cols else 0
            self.stage1_ws = torch.empty(ws1, device=dev, dtype=torch.uint8) if ws1 else None
            if self.k0 > k:
                ws2 = lib.atk_select_workspace_bytes(code, 1, self.k0, k)
                self.select_ws = torch.empty(ws2, device=dev, dtype=torch.uint8) if ws2 else None
                self.values = torch.empty(k, device=dev, dtype=dtype)
                self.indices = torch.empty(k, device=dev, dtype=torch.int64)
            else:
                self.select_ws = None
                self.values, self.indices = self.cand_vals[:k], self.cand_idx[:k]

    def _init_push(self, block: int, esize: int) -> None:
        """Two sets of dense candidate arrays in one shared buffer, the peers' mappings of
        theirs, and the argument arrays of the push for either set."""
        import ctypes

        dev, world, rank = self.device, self.world, self.rank
        idx_bytes = (block * world * 8 + 255) // 256 * 256
        val_bytes = (block * world * esize + 255) // 256 * 256
        set_bytes = idx_bytes + val_bytes
        self._shared = PeerBuffers(2 * set_bytes, dev, self.group)
        self._recv = self._shared.local
        self._flag = torch.zeros(1, device=dev, dtype=torch.float32)
        self._sets = []
        mine = self.cols * self.j                                  # real candidates of this rank
        for s in range(2):
            base = s * set_bytes
            cand_idx = self._recv[base:base + block * world * 8].view(torch.int64)
            cand_vals = self._recv[base + idx_bytes:base + idx_bytes + block * world * esize].view(self.dtype)
            local_idx = cand_idx[rank * block:rank * block + mine]
            local_vals = cand_vals[rank * block:rank * block + mine]
            others = [r for r in range(world) if r != rank]
            src = (ctypes.c_void_p * 2)(local_idx.data_ptr(), local_vals.data_ptr())
            nbytes = (ctypes.c_size_t * 2)(mine * 8, mine * esize)
            dst = (ctypes.c_void_p * (2 * len(others)))()
            for d, r in enumerate(others):
                peer = self._shared.ptrs[r] + base
                dst[d] = peer + rank * block * 8
                dst[len(others) + d] = peer + idx_bytes + rank * block * esize
            self._sets.append({"cand_idx": cand_idx, "cand_vals": cand_vals, "local_idx": local_idx,
                               "local_vals": local_vals, "push": (src, nbytes, len(others), dst)})
        self._use_set(0)

    def _use_set(self, s: int) -> None:
        cur = self._sets[s]
        self.cand_idx, self.cand_vals = cur["cand_idx"], cur["cand_vals"]
        self.local_idx, self.local_vals = cur["local_idx"], cur["local_vals"]
        self._push_args = cur["push"]

    def close(self) -> None:
        """Collective tear-down of the buffers shared with the peers (``"push"`` only)."""
        shared = getattr(self, "_shared", None)
        if shared is not None:
            self._sets, self._recv, self.cand_idx, self.cand_vals = [], None, None, None
            self.local_idx, self.local_vals = None, None
            if self.k0 <= self.k:                 # the results were views of the shared buffer
                self.values, self.indices = None, None
            shared.close()
            self._shared = None

    def __call__(self, slab: Tensor, events: list | None = None) -> tuple[Tensor, Tensor]:
        if slab.ndim != 2 or tuple(slab.shape) != (self.stripes, self.cols) or slab.dtype != self.dtype:
            raise ValueError(f"slab must be {self.stripes} x {self.cols} of {self.dtype}, got "
                             f"{tuple(slab.shape)} of {slab.dtype}")

        def mark():
            if events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(torch.cuda.current_stream(self.device))
                events.append(ev)

        if self.exchange == "push":
            self._use_set(self._step & 1)
            self._step += 1
        if self.cols:
            _native_stage1_slab(slab, self.total_buckets, self.start, self.j,
                                out=(self.local_vals[:self.cols * self.j], self.local_idx[:self.cols * self.j]),
                                workspace=self.stage1_ws)
        mark()
        if self.exchange == "push":
            src, nbytes, n_dst, dst = self._push_args
            with torch.cuda.device(self.device):
                _native.check(_native.lib().atk_push_blocks(2, src, nbytes, n_dst, dst,
                                                            _native.current_stream_ptr(self.device)))
            # orders the streams: when it ends here, every rank's push kernel has ended
            dist.all_reduce(self._flag, group=self.group)
        elif self.world > 1:
            # rank g's block is slots [g*block, (g+1)*block); real columns fill the
            # gathered buffer from the front, so its first k0 slots are the candidates
            dist.all_gather_into_tensor(self._packed_all, self._packed_local, group=self.group)
            blocks = self._packed_all.view(self.world, self._block_bytes)
            esize = self.local_vals.element_size()
            self.cand_idx.view(self.world, self.block).copy_(blocks[:, :self._idx_bytes].view(torch.int64))
            self.cand_vals.view(self.world, self.block).copy_(
                blocks[:, self._idx_bytes:self._idx_bytes + self.block * esize].view(self.dtype))
        mark()
        if self.k0 > self.k:
            _native_select(self.cand_vals[:self.k0], self.cand_idx[:self.k0], self.k,
                           out=(self.values, self.indices), workspace=self.select_ws)
        elif self.exchange == "push":             # nothing to select: the candidates of this step's set
            self.values, self.indices = self.cand_vals[:self.k], self.cand_idx[:self.k]
        mark()
        return self.values, self.indices


def topk_long_row(
    slab: Tensor,
    k: int,
    j: int,
    k_mult: int,
    group: dist.ProcessGroup | None = None,
    stage1: Callable[[Tensor, int, int, int], tuple[Tensor, Tensor]] | None = None,
    select: Callable[[Tensor, Tensor, int], tuple[Tensor, Tensor]] | None = None,
) -> tuple[Tensor, Tensor]:
    """Approximate top-k of one long interleaved row sharded by bucket groups.

    :param slab: this rank's dense ``stripes x cols`` slab (columns
        :func:`bucket_group` of the ``stripes x b`` view, ``b = k*k_mult/j``).
    :returns: the ``k`` selected ``(values, indices)``, identical on every rank
        and identical to the single-GPU result; indices are positions in the
        full row.

    ``stage1`` / ``select`` default to the native kernels; they are parameters so
    that the partitioning and the exchange can be exercised on CPU ranks.  For a
    step that is repeated (or captured in a CUDA graph) use :class:`LongRowTopK`,
    which allocates its buffers once.
    """
    if k_mult < 1:
        raise ValueError(f"k_mult must be >=1, was {k_mult}")
    k0 = k * k_mult
    if k0 % j:
        raise RuntimeError("topk: j must divide k")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    total_buckets = k0 // j
    start, stop = bucket_group(total_buckets, rank, world)
    if slab.ndim != 2 or slab.shape[1] != stop - start:
        raise ValueError(f"slab must be stripes x {stop - start}, got {tuple(slab.shape)}")
    stage1 = stage1 or _native_stage1_slab
    select = select or _native_select

    block = group_width(total_buckets, world) * j
    if stop > start:
        local_vals, local_idx = stage1(slab, total_buckets, start, j)
    else:
        local_vals = torch.empty(0, device=slab.device, dtype=slab.dtype)
        local_idx = torch.empty(0, device=slab.device, dtype=torch.int64)
    if world > 1:
        if local_vals.numel() < block:           # a short (or empty) last group: pad its block
            pad = block - local_vals.numel()
            local_vals = torch.cat([local_vals, local_vals.new_zeros(pad)])
            local_idx = torch.cat([local_idx, local_idx.new_full((pad,), -1)])
        cand_vals = torch.empty(block * world, device=slab.device, dtype=slab.dtype)
        cand_idx = torch.empty(block * world, device=slab.device, dtype=torch.int64)
        # rank g's candidates are slots [g*block, (g+1)*block): a plain all-gather;
        # the padding of short groups lands behind the k0 real candidates
        dist.all_gather_into_tensor(cand_vals, local_vals, group=group)
        dist.all_gather_into_tensor(cand_idx, local_idx, group=group)
        cand_vals, cand_idx = cand_vals[:k0], cand_idx[:k0]
    else:
        cand_vals, cand_idx = local_vals, local_idx
    if k0 == k:
        return cand_vals, cand_idx
    return select(cand_vals, cand_idx, k)
