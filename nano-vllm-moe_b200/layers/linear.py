"""Tensor-parallel linear layers that own the FP8 buffers and call the quant method.

Interface-compatible with the reference's nanovllm/layers/linear.py:15-262
(constructor arguments, ``weight_loader`` shard ids, ``tp_dim``/``tp_rank``/
``tp_size`` attributes, ``get_quant_output_offset_size``), so the reference's
model files and checkpoint loader can use these classes unchanged.

Column-parallel layers split the output channels (N) across the TP group and
need no communication; the row-parallel layer splits K, adds the bias on rank
0 only and sums the per-rank bf16 outputs with an NCCL all-reduce.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from ..quantization.base_config import QuantizeMethodBase


def divide(numerator: int, denominator: int) -> int:
    if numerator % denominator != 0:
        raise AssertionError(f"{numerator} is not divisible by {denominator}")
    return numerator // denominator


def _group_size_rank(group) -> tuple[int, int]:
    if group is not None:
        return dist.get_world_size(group), dist.get_rank(group)
    if dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


class LinearBase(nn.Module):
    def __init__(self, input_size: int, output_size: int, tp_dim: int | None = None,
                 tp_group: Optional[dist.ProcessGroup] = None,
                 quant_method: QuantizeMethodBase | None = None, **kwargs):
        super().__init__()
        self.input_size = input_size
        self.output_size = output_size
        self.tp_dim = tp_dim
        self.tp_group = tp_group
        self.quant_method = quant_method
        self.tp_size, self.tp_rank = _group_size_rank(tp_group)

    def is_quantized(self) -> bool:
        return self.quant_method is not None

    def apply_linear(self, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if self.quant_method is None:
            return F.linear(x, self.weight, bias)
        return self.quant_method.apply(self, x, bias)

    def _make_params(self, k_part: int, n_parts: list[int], bias: bool) -> None:
        n_part = sum(n_parts)
        if self.quant_method is None:
            self.weight = nn.Parameter(torch.empty(n_part, k_part))
            self.weight.weight_loader = self.weight_loader
        else:
            self.quant_method.create_weights(
                self, input_size_per_partition=k_part, output_partition_sizes=n_parts,
                input_size=self.input_size, output_size=self.output_size,
                params_dtype=torch.get_default_dtype())
        if bias:
            self.bias = nn.Parameter(torch.empty(n_part))
            self.bias.weight_loader = self.weight_loader
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # pragma: no cover - abstract
        raise NotImplementedError


class ReplicatedLinear(LinearBase):
    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 tp_group: Optional[dist.ProcessGroup] = None, **kwargs):
        super().__init__(input_size, output_size, tp_group=tp_group, **kwargs)
        self.quant_method = None
        self._make_params(input_size, [output_size], bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        param.data.copy_(loaded_weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight, self.bias)


class ColumnParallelLinear(LinearBase):
    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 tp_group: Optional[dist.ProcessGroup] = None,
                 quant_method: QuantizeMethodBase | None = None, **kwargs):
        super().__init__(input_size, output_size, 0, tp_group=tp_group, quant_method=quant_method, **kwargs)
        self.input_size_per_partition = input_size
        self.output_size_per_partition = divide(output_size, self.tp_size)
        self._make_params(input_size, [self.output_size_per_partition], bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        rows = param.data.size(self.tp_dim)
        param.data.copy_(loaded_weight.narrow(self.tp_dim, self.tp_rank * rows, rows))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.apply_linear(x, self.bias)


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel projections fused along N (gate_up): shard ids 0, 1, ..."""

    def __init__(self, input_size: int, output_sizes: list[int], bias: bool = False,
                 tp_group: Optional[dist.ProcessGroup] = None,
                 quant_method: QuantizeMethodBase | None = None, **kwargs):
        self.output_sizes = list(output_sizes)
        super().__init__(input_size, sum(output_sizes), bias=bias, tp_group=tp_group,
                         quant_method=quant_method, **kwargs)
        if self.quant_method is not None:
            self.output_partition_sizes = [s // self.tp_size for s in self.output_sizes]

    def get_quant_output_offset_size(self, loaded_shard_id: int) -> tuple[int, int]:
        offset = sum(self.output_sizes[:loaded_shard_id]) // self.tp_size
        return offset, self.output_sizes[loaded_shard_id] // self.tp_size

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: int):
        offset, size = self.get_quant_output_offset_size(loaded_shard_id)
        mine = loaded_weight.chunk(self.tp_size, self.tp_dim)[self.tp_rank]
        param.data.narrow(self.tp_dim, offset, size).copy_(mine)


class QKVParallelLinear(ColumnParallelLinear):
    """q, k and v projections fused along N and split by heads: shard ids "q", "k", "v"."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int,
                 total_num_kv_heads: int | None = None, bias: bool = False,
                 tp_group: Optional[dist.ProcessGroup] = None,
                 quant_method: QuantizeMethodBase | None = None, **kwargs):
        self.head_size = head_size
        self.total_num_heads = total_num_heads
        self.total_num_kv_heads = total_num_kv_heads or total_num_heads
        tp_size, _ = _group_size_rank(tp_group)
        self.num_heads = divide(self.total_num_heads, tp_size)
        self.num_kv_heads = divide(self.total_num_kv_heads, tp_size)
        output_size = (self.total_num_heads + 2 * self.total_num_kv_heads) * head_size
        super().__init__(hidden_size, output_size, bias=bias, tp_group=tp_group,
                         quant_method=quant_method, **kwargs)

    def get_quant_output_offset_size(self, loaded_shard_id: str) -> tuple[int, int]:
        q = self.num_heads * self.head_size
        kv = self.num_kv_heads * self.head_size
        try:
            return {"q": (0, q), "k": (q, kv), "v": (q + kv, kv)}[loaded_shard_id]
        except KeyError:
            raise AssertionError(f"shard id must be 'q', 'k' or 'v', got {loaded_shard_id!r}") from None

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: str):
        offset, size = self.get_quant_output_offset_size(loaded_shard_id)
        mine = loaded_weight.chunk(self.tp_size, self.tp_dim)[self.tp_rank]
        param.data.narrow(self.tp_dim, offset, size).copy_(mine)


class RowParallelLinear(LinearBase):
    def __init__(self, input_size: int, output_size: int, bias: bool = False, reduce_results: bool = True,
                 tp_group: Optional[dist.ProcessGroup] = None,
                 quant_method: QuantizeMethodBase | None = None, **kwargs):
        super().__init__(input_size, output_size, 1, tp_group=tp_group, quant_method=quant_method, **kwargs)
        self.input_size_per_partition = divide(input_size, self.tp_size)
        self.output_size_per_partition = output_size
        self.reduce_results = reduce_results
        self._make_params(self.input_size_per_partition, [output_size], bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        if param.data.dim() == 1:           # bias: replicated, added on rank 0 only
            param.data.copy_(loaded_weight)
            return
        cols = param.data.size(self.tp_dim)
        param.data.copy_(loaded_weight.narrow(self.tp_dim, self.tp_rank * cols, cols))

    # Optional: from this many rows on, cut the row-parallel forward into chunks so that the
    # all-reduce of chunk i (second stream) runs under the GEMM of chunk i+1.  Off by default:
    # measured on 2 B200s at M=4096 it is slower than GEMM + one all-reduce replayed from a CUDA
    # graph (four 7 MB all-reduces cost more than one 29 MB one, and the eager launches are
    # host-bound); kept for large eager prefills.
    overlap_min_rows = None
    overlap_chunks = 4

    # Fold the all-reduce into the GEMM through peer memory (torch symmetric memory on the TP group), two forms:
    #  * reduce-scatter + all-gather ("rs", what "auto" takes from peer_reduce_min_rows rows and K/tp >= peer_rs_min_k):
    #    the epilogue TMA-stores the rows of band r only into rank r's slot buffer while the GEMM runs; after a
    #    symmetric-memory barrier rank r adds the tp partials of its band (fp32, rank order) and stores the reduced
    #    band into every rank's output; a second barrier.  A rank sends 2 (tp - 1) / tp of the payload.
    #    `reduce_results="scatter"` stops after the sum and returns this rank's band of rows only (for a caller that
    #    continues row-sharded).  Measured on 2 B200s at M = 16384: o_proj (K/tp = 1792) 254 us against 363 us with the
    #    NCCL all-reduce, down (K/tp = 9472) 679 us against 796 us.
    #  * store-to-everyone (True): every rank's epilogue stores its whole partial into its slot of every rank's buffer,
    #    one barrier, every rank sums locally.  (tp - 1) times the payload per rank: only sensible between two ranks
    #    (down at M = 16384: 697 us).
    # False = always the NCCL all-reduce, as the reference.
    # defer_gather (reduce-scatter form only): forward returns once the GEMM (with its scatter) is enqueued; the
    # barrier, the sum and the all-gather run on a side stream, so that the caller's next kernels -- work that does not
    # read this output, e.g. the next micro-batch's or an independent linear's GEMM -- run while NVLink carries the
    # reduced bands.  The output must not be read before `wait_reduce()` (which makes the current stream wait for
    # the side stream); the layer's own next call waits by itself.
    # peer_scatter: how the partial bands reach their owners.  "epilogue" = the GEMM's TMA stores (the transfer
    # overlaps the GEMM's own tiles: right when the local GEMM outlasts the transfer); "copy" = the GEMM writes a local
    # partial result and the copy engines push its bands to the peers afterwards (large NVLink packets, no SM work;
    # with defer_gather the whole exchange runs beside the caller's next kernels: right when K/tp is short and the
    # transfer would outlast the GEMM); "auto" picks by that comparison.
    defer_gather = False
    peer_scatter = "auto"
    peer_reduce = "auto"
    peer_reduce_min_rows = 512
    peer_reduce_min_k = 4096
    peer_rs_min_k = 0

    def _use_peer_rs(self, x: torch.Tensor, rows: int) -> bool:
        """Reduce-scatter + all-gather through peer memory (more than two ranks, or forced with peer_reduce = "rs")."""
        if self.peer_reduce is False or getattr(self, "_peer_failed", False):
            return False
        if not (x.is_cuda and x.dtype == torch.bfloat16 and getattr(self, "_fp8_backend", None) == "fp8lin_w8a8"):
            return False
        if self.output_size % 8:
            return False
        if self.peer_reduce == "rs" or self.reduce_results == "scatter":
            wanted = True
        elif self.peer_reduce == "auto":
            wanted = rows >= self.peer_reduce_min_rows and self.input_size_per_partition >= self.peer_rs_min_k
        else:
            wanted = False                  # True = the store-to-everyone form at any number of ranks
        return wanted and (getattr(self, "_rs_cap", 0) >= rows or not torch.cuda.is_current_stream_capturing())

    def _rs_buffers(self, rows: int, device):
        import torch.distributed._symmetric_memory as symm
        cap = getattr(self, "_rs_cap", 0)
        if cap < rows:
            cap = max(rows, 2 * cap)
            band = -(-(-(-cap // self.tp_size)) // 32) * 32             # rows per band, a multiple of 32
            n = self.output_size
            group = self.tp_group if self.tp_group is not None else dist.group.WORLD
            # [tp slots of one band | the whole output]: peers store partial bands into the slots and reduced bands into the output
            buf = symm.empty((self.tp_size * band + cap) * n, dtype=torch.bfloat16, device=device)
            self._rs_handle = symm.rendezvous(buf, group)
            self._rs_buf, self._rs_cap, self._rs_band_cap = buf, cap, band
        return self._rs_buf, self._rs_handle

    def _forward_peer_rs(self, x: torch.Tensor, bias, rows: int) -> torch.Tensor:
        from ..quantization import kernels
        x2 = x.reshape(rows, x.shape[-1])
        buf, handle = self._rs_buffers(rows, x.device)
        n, tp, rank = self.output_size, self.tp_size, self.tp_rank
        band = -(-(-(-rows // tp)) // 32) * 32
        band_cap = self._rs_band_cap
        slot_elems = band_cap * n
        y_off = tp * slot_elems                                  # element offset of the output inside the buffer
        # the previous call's second barrier guarantees that every rank has summed its slots and read its output
        self.wait_reduce()                                       # a deferred gather of the previous call still owns the buffers
        mine = max(0, min(band, rows - rank * band))
        by_copy = self.peer_scatter == "copy" or (
            self.peer_scatter == "auto" and self.reduce_results != "scatter"
            # GEMM time ~ 2 M K' N / 2.2e15 against (tp - 1) / tp * 2 M N bytes at ~0.6 TB/s of NVLink writes
            and self.input_size_per_partition < 3667 * (tp - 1) // tp)
        if by_copy:
            return self._finish_rs_by_copy(x, x2, bias, rows, band, mine, buf, handle, slot_elems, y_off)
        dst = [int(handle.buffer_ptrs[r]) + rank * slot_elems * 2 for r in range(tp)]
        kernels.launch_w8a8_reduce_scatter(x2, self.qweight_packed, self.input_scale, self.weight_scale, bias, dst, n, band)
        if self.reduce_results == "scatter":
            handle.barrier(channel=0)                            # every rank's partial rows of my band have landed
            out = torch.empty((mine, n), dtype=torch.bfloat16, device=x.device)
            kernels.sum_slots_gather(buf.data_ptr(), tp, slot_elems, n, [out.data_ptr()], n, 0, mine, n, x.device)
            handle.barrier(channel=1)
            return out
        ys = [int(handle.buffer_ptrs[r]) + y_off * 2 for r in range(tp)]
        y = buf[y_off:y_off + rows * n].view(rows, n)            # (valid until this layer's next call)

        def second_half():
            handle.barrier(channel=0)                            # every rank's partial rows of my band have landed
            kernels.sum_slots_gather(buf.data_ptr(), tp, slot_elems, n, ys, n, rank * band, mine, n, x.device)
            handle.barrier(channel=1)                            # every band of the result is in place everywhere

        if not self.defer_gather:
            second_half()
            return y.view(*x.shape[:-1], n)
        main = torch.cuda.current_stream(x.device)
        side = self._exchange_stream(x.device)
        scattered = torch.cuda.Event()
        scattered.record(main)
        with torch.cuda.stream(side):
            side.wait_event(scattered)
            second_half()
            done = torch.cuda.Event()
            done.record(side)
        self._pending_gather = done
        return y.view(*x.shape[:-1], n)

    def _finish_rs_by_copy(self, x, x2, bias, rows, band, mine, buf, handle, slot_elems, y_off):
        """Reduce-scatter with the copy engines: the plain GEMM writes this rank's partial result locally, then band r
        goes to rank r's slot by one peer-to-peer copy each, the owner sums, and the reduced band is stored to every
        rank.  With defer_gather everything after the GEMM runs on the side stream."""
        from ..quantization import kernels
        n, tp, rank = self.output_size, self.tp_size, self.tp_rank
        part = getattr(self, "_partial", None)
        if part is None or part.shape[0] < rows:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the row-parallel partial buffer must exist before a CUDA graph capture: run the shape once first")
            part = self._partial = torch.empty((max(rows, getattr(self, "_rs_cap", rows)), n), dtype=torch.bfloat16, device=x.device)
        self.quant_method.apply(self, x2, bias, out=part[:rows])
        ys = [int(handle.buffer_ptrs[r]) + y_off * 2 for r in range(tp)]
        y = buf[y_off:y_off + rows * n].view(rows, n)

        def exchange():
            for step in range(tp):
                r = (rank + step) % tp                           # every rank starts with a different peer
                lo, hi = r * band, min(rows, (r + 1) * band)
                if hi > lo:
                    slot = handle.get_buffer(r, (hi - lo, n), torch.bfloat16, storage_offset=rank * slot_elems)
                    slot.copy_(part[lo:hi], non_blocking=True)
            handle.barrier(channel=0)
            kernels.sum_slots_gather(buf.data_ptr(), tp, slot_elems, n, ys, n, rank * band, mine, n, x.device)
            handle.barrier(channel=1)

        if not self.defer_gather:
            exchange()
            return y.view(*x.shape[:-1], n)
        main = torch.cuda.current_stream(x.device)
        side = self._exchange_stream(x.device)
        computed = torch.cuda.Event()
        computed.record(main)
        with torch.cuda.stream(side):
            side.wait_event(computed)
            exchange()
            done = torch.cuda.Event()
            done.record(side)
        self._pending_gather = done
        return y.view(*x.shape[:-1], n)

    _exchange_streams: dict = {}

    @classmethod
    def _exchange_stream(cls, device) -> torch.cuda.Stream:
        """One side stream per device for ALL row-parallel layers: their deferred exchanges (each a sequence of
        cross-rank barriers) then run in the same order on every rank, whatever the hardware does with parallel
        branches -- two layers' barrier kernels can never wait for each other crosswise."""
        key = device.index if device.index is not None else torch.cuda.current_device()
        st = cls._exchange_streams.get(key)
        if st is None:
            st = cls._exchange_streams[key] = torch.cuda.Stream(device)
        return st

    def wait_reduce(self) -> None:
        """Make the current stream wait for a deferred gather of this layer's last call (no-op otherwise)."""
        done = getattr(self, "_pending_gather", None)
        if done is not None:
            torch.cuda.current_stream().wait_event(done)
            self._pending_gather = None

    def _use_peer_reduce(self, x: torch.Tensor, rows: int) -> bool:
        if self.peer_reduce is False or self.peer_reduce == "rs" or getattr(self, "_peer_failed", False):
            return False
        if self.peer_reduce == "auto" and self.tp_size > 2:
            return False                    # store-to-everyone only pays between two ranks
        if not (x.is_cuda and x.dtype == torch.bfloat16 and getattr(self, "_fp8_backend", None) == "fp8lin_w8a8"):
            return False
        if rows < self.peer_reduce_min_rows or self.output_size % 8:
            return False
        if self.peer_reduce == "auto" and self.input_size_per_partition < self.peer_reduce_min_k:
            return False
        # the peer buffers must exist before a stream capture starts
        return getattr(self, "_peer_cap", 0) >= rows or not torch.cuda.is_current_stream_capturing()

    def _peer_buffers(self, rows: int, device):
        import torch.distributed._symmetric_memory as symm
        cap = getattr(self, "_peer_cap", 0)
        if cap < rows:
            cap = max(rows, 2 * cap)
            group = self.tp_group if self.tp_group is not None else dist.group.WORLD
            buf = symm.empty((self.tp_size, cap, self.output_size), dtype=torch.bfloat16, device=device)
            self._peer_handle = symm.rendezvous(buf, group)
            self._peer_buf, self._peer_cap = buf, cap
        return self._peer_buf, self._peer_handle, cap

    def _forward_peer_reduce(self, x: torch.Tensor, bias, rows: int) -> torch.Tensor:
        from ..quantization import kernels
        x2 = x.reshape(rows, x.shape[-1])
        buf, handle, cap = self._peer_buffers(rows, x.device)
        slot_bytes = cap * self.output_size * 2
        dst = [int(handle.buffer_ptrs[r]) + self.tp_rank * slot_bytes for r in range(self.tp_size)]
        handle.barrier(channel=0)                       # nobody is still summing the previous call's slots
        kernels.launch_w8a8_scatter(x2, self.qweight_packed, self.input_scale, self.weight_scale, bias, dst, self.output_size)
        handle.barrier(channel=1)                       # every rank's partial tiles have landed everywhere
        y = kernels.sum_slots(buf, rows, self.output_size)
        return y.view(*x.shape[:-1], self.output_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bias = self.bias if self.tp_rank == 0 else None
        reduce = self.tp_size > 1 and bool(self.reduce_results)
        rows = x.numel() // x.shape[-1] if x.dim() > 0 else 0
        if reduce and (self._use_peer_rs(x, rows) or self._use_peer_reduce(x, rows)):
            try:
                if self._use_peer_rs(x, rows):
                    return self._forward_peer_rs(x, bias, rows)
                return self._forward_peer_reduce(x, bias, rows)
            except (RuntimeError, ImportError, AttributeError) as exc:
                if self.peer_reduce in (True, "rs") or getattr(self, "_peer_cap", 0) > 0 or getattr(self, "_rs_cap", 0) > 0:
                    raise
                # symmetric memory is not available for this group (every rank fails alike in the
                # collective rendezvous): remember it and use the all-reduce from now on
                self._peer_failed = True
                import warnings
                warnings.warn(f"row-parallel peer reduction unavailable, using all-reduce: {exc}")
        if (reduce and self.quant_method is not None and x.is_cuda and x.dtype == torch.bfloat16
                and self.overlap_min_rows is not None and rows >= self.overlap_min_rows
                and not torch.cuda.is_current_stream_capturing()):
            return self._forward_overlapped(x, bias, rows)
        y = self.apply_linear(x, bias)
        if reduce:
            dist.all_reduce(y, group=self.tp_group)
        return y

    def _forward_overlapped(self, x: torch.Tensor, bias, rows: int) -> torch.Tensor:
        """GEMM and all-reduce pipelined over row chunks: same sums as the one-shot form (the
        reduction is elementwise), but only the last chunk's all-reduce is exposed."""
        x2 = x.reshape(rows, x.shape[-1])
        y = torch.empty((rows, self.output_size), dtype=torch.bfloat16, device=x.device)
        compute = torch.cuda.current_stream(x.device)
        comm = getattr(self, "_comm_stream", None)
        if comm is None:
            comm = self._comm_stream = torch.cuda.Stream(x.device)
        step = -(-rows // self.overlap_chunks)
        step = (step + 127) // 128 * 128
        for r0 in range(0, rows, step):
            r1 = min(rows, r0 + step)
            part = y[r0:r1]
            self.quant_method.apply(self, x2[r0:r1], bias, out=part)
            done = torch.cuda.Event()
            done.record(compute)
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                dist.all_reduce(part, group=self.tp_group)
        compute.wait_stream(comm)
        y.record_stream(comm)
        return y.view(*x.shape[:-1], self.output_size)
