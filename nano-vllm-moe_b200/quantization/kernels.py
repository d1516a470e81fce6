"""Functional launchers over the C ABI — the calls ``Fp8LinearMethod.apply`` makes.

They take torch CUDA tensors, pass raw device pointers and the current CUDA
stream to ``libfp8lin.so`` and return the bf16 result.  Counterparts in the
reference: ``launch_w8a16_gemm`` (nanovllm/quantization/kernels/fp8.py:79-109),
``launch_w8a8_cuda_ptx_jit`` (w8a8_jit.py:521-542), ``launch_w8a8_cutlass_gemm``
(cuda_ext.py:84-106), ``quantize_activation_w8a8`` (kernels/fp8.py:263-268).
Unlike the reference there is one backend and no environment-variable dispatch;
the kernel variant is a pure function of (scheme, M, K, N).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib

_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_retired: list[torch.Tensor] = []       # outgrown scratch buffers, kept alive (see workspace())


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("fp8lin kernels need CUDA tensors (there is no CPU path)")


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch for the current stream of ``device``, grown on demand.

    One buffer per (device, stream): calls on different streams never share scratch.
    A buffer that is outgrown is retired, not freed: a CUDA graph captured earlier has its
    address (split-K counters, partial sums, quantised activations) baked in, and its replays
    must keep writing into memory nobody else owns.  ``release_workspaces()`` frees everything
    once no such graph is left.

    Growing allocates and zero-fills, which must not happen inside a stream capture: warm every
    shape up once (or call ``reserve_workspace`` with the largest size) ON THE STREAM THAT WILL
    CAPTURE, before the capture starts.  ``torch.cuda.graph`` captures on a side stream, so the
    warm-up belongs inside ``with torch.cuda.stream(side):`` too.  Graphs captured on the same
    stream share one scratch buffer; replay them on one stream at a time."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream_ptr(device))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                f"fp8lin scratch for this stream must grow to {nbytes} bytes during a CUDA graph capture; "
                "run the shape once (or call reserve_workspace) on the capturing stream before the capture")
        size = max(nbytes, _lib.WS_HEADER_BYTES)
        if ws is not None:
            size = max(size, 2 * ws.numel())
            _retired.append(ws)
        ws = torch.zeros(size, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def reserve_workspace(device: torch.device, nbytes: int) -> None:
    """Make the current stream's scratch at least ``nbytes`` large (see ``workspace``)."""
    workspace(device, nbytes)


def release_workspaces() -> None:
    """Free every scratch buffer, retired ones included.  Only when no kernel of this library is
    in flight and no CUDA graph that captured one of its calls will be replayed again."""
    torch.cuda.synchronize()
    _workspaces.clear()
    _retired.clear()


def workspace_bytes(scheme: int, m: int, k: int, n: int) -> int:
    return int(_lib.load().fp8lin_workspace_bytes(scheme, m, k, n))


def launch_count() -> int:
    """Kernel launches the library has made so far in this process (difference it around a call)."""
    return int(_lib.load().fp8lin_launch_count())


def variant_name(scheme: int, m: int, k: int, n: int) -> str:
    return _lib.load().fp8lin_variant_name(scheme, m, k, n).decode()


def set_tuning(knob: str, value: int) -> None:
    _lib.raise_for(_lib.load().fp8lin_set_tuning(knob.encode(), int(value)), "fp8lin_set_tuning")


def read_status(device: torch.device) -> int:
    """Blocking check of the device status word of the current stream's scratch."""
    ws = workspace(device, _lib.WS_HEADER_BYTES)
    out = ctypes.c_int(0)
    rc = _lib.load().fp8lin_read_status(ws.data_ptr(), _stream_ptr(device), ctypes.byref(out))
    _lib.raise_for(rc, "fp8lin_read_status")
    return out.value


def packed_bytes(k: int, n: int) -> int:
    return int(_lib.load().fp8lin_packed_bytes(k, n))


def _pack(src: torch.Tensor, k: int, n: int, from_kn: bool) -> torch.Tensor:
    _require_cuda(src)
    if src.dtype not in (torch.uint8, torch.float8_e4m3fn) or src.dim() != 2:
        raise ValueError("weight codes must be a 2-D uint8/float8_e4m3fn tensor")
    src = src.contiguous()
    out = torch.empty(packed_bytes(k, n), dtype=torch.uint8, device=src.device)
    fn = _lib.load().fp8lin_prepack_weight if from_kn else _lib.load().fp8lin_pack_weight_nk
    with torch.cuda.device(src.device):
        rc = fn(src.data_ptr(), out.data_ptr(), k, n, _stream_ptr(src.device))
    _lib.raise_for(rc, "fp8lin_prepack_weight" if from_kn else "fp8lin_pack_weight_nk")
    return out


def prepack_weight(qweight_kn: torch.Tensor) -> torch.Tensor:
    """e4m3 codes [K, N] (the reference's ``qweight`` buffer) -> the kernels' packed tile layout."""
    k, n = qweight_kn.shape
    return _pack(qweight_kn, k, n, True)


def pack_weight_nk(qweight_nk: torch.Tensor) -> torch.Tensor:
    """e4m3 codes [N, K] (the checkpoint layout) -> the kernels' packed tile layout."""
    n, k = qweight_nk.shape
    return _pack(qweight_nk, k, n, False)


def _check_linear_args(x, w_packed, weight_scale, bias):
    _require_cuda(x, w_packed, weight_scale, bias)
    if x.dim() != 2 or x.dtype != torch.bfloat16:
        raise ValueError("x must be a 2-D bfloat16 tensor [M, K]")
    if w_packed.dtype != torch.uint8 or w_packed.dim() != 1 or not w_packed.is_contiguous():
        raise ValueError("w_packed must be the flat uint8 buffer made by prepack_weight / pack_weight_nk")
    if weight_scale.dtype != torch.float32 or weight_scale.dim() != 1:
        raise ValueError("weight_scale must be float32 with one value per output channel")
    n, k = weight_scale.numel(), x.shape[1]
    if k % 16 != 0 or w_packed.numel() != packed_bytes(k, n):
        raise ValueError(f"x has K={k}, weight_scale has N={n}, but the packed weight holds "
                         f"{w_packed.numel()} bytes (expected {packed_bytes(k, n) if k % 16 == 0 else 'K % 16 == 0'})")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != n):
        raise ValueError("bias must be bfloat16 [N]")
    if x.stride(1) != 1:
        x = x.contiguous()
    return x, n, k


def launch_w8a16_gemm(x: torch.Tensor, w_packed: torch.Tensor, weight_scale: torch.Tensor,
                      bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 ``(x @ W^T) * weight_scale + bias`` with packed e4m3 weights."""
    x, n, k = _check_linear_args(x, w_packed, weight_scale, bias)
    m = x.shape[0]
    y = out if out is not None else torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        need = workspace_bytes(_lib.W8A16, m, k, n)
        ws = workspace(x.device, need)
        rc = _lib.load().fp8lin_w8a16(
            x.data_ptr(), x.stride(0), w_packed.data_ptr(), weight_scale.data_ptr(),
            bias.data_ptr() if bias is not None else None, y.data_ptr(), y.stride(0),
            m, k, n, ws.data_ptr(), ws.numel(), _stream_ptr(x.device))
    _lib.raise_for(rc, "fp8lin_w8a16")
    return y


def launch_w8a8_gemm(x: torch.Tensor, w_packed: torch.Tensor, input_scale: torch.Tensor,
                     weight_scale: torch.Tensor, bias: torch.Tensor | None = None,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """Static-scale W8A8: x is quantised to e4m3 with ``input_scale`` inside the call."""
    x, n, k = _check_linear_args(x, w_packed, weight_scale, bias)
    _require_cuda(input_scale)
    if input_scale.dtype != torch.float32 or input_scale.numel() != 1:
        raise ValueError("input_scale must be one float32 value on the device")
    m = x.shape[0]
    y = out if out is not None else torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        need = workspace_bytes(_lib.W8A8_STATIC, m, k, n)
        ws = workspace(x.device, need)
        rc = _lib.load().fp8lin_w8a8(
            x.data_ptr(), x.stride(0), w_packed.data_ptr(), weight_scale.data_ptr(), input_scale.data_ptr(),
            bias.data_ptr() if bias is not None else None, y.data_ptr(), y.stride(0),
            m, k, n, ws.data_ptr(), ws.numel(), _stream_ptr(x.device))
    _lib.raise_for(rc, "fp8lin_w8a8")
    return y


def launch_w8a8_preq(xq: torch.Tensor, w_packed: torch.Tensor, input_scale: torch.Tensor, weight_scale: torch.Tensor,
                     bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """W8A8 linear on activations that are already e4m3 codes (uint8 [M, K], contiguous), e.g. from
    ``rmsnorm_quant``: no quantiser pass."""
    _require_cuda(xq, w_packed, weight_scale, input_scale, bias)
    if xq.dtype != torch.uint8 or xq.dim() != 2 or not xq.is_contiguous():
        raise ValueError("xq must be a contiguous 2-D uint8 tensor of e4m3 codes [M, K]")
    m, k = xq.shape
    n = weight_scale.numel()
    if k % 16 != 0 or w_packed.numel() != packed_bytes(k, n):
        raise ValueError(f"xq has K={k}, weight_scale has N={n}, but the packed weight holds {w_packed.numel()} bytes")
    y = out if out is not None else torch.empty((m, n), dtype=torch.bfloat16, device=xq.device)
    with torch.cuda.device(xq.device):
        ws = workspace(xq.device, workspace_bytes(_lib.W8A8_STATIC, m, k, n))
        rc = _lib.load().fp8lin_w8a8_preq(
            xq.data_ptr(), w_packed.data_ptr(), weight_scale.data_ptr(), input_scale.data_ptr(),
            bias.data_ptr() if bias is not None else None, y.data_ptr(), y.stride(0), m, k, n,
            ws.data_ptr(), ws.numel(), _stream_ptr(xq.device))
    _lib.raise_for(rc, "fp8lin_w8a8_preq")
    return y


def rmsnorm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float, input_scale: torch.Tensor | None = None,
                  residual: torch.Tensor | None = None, want_bf16: bool = False,
                  xq_out: torch.Tensor | None = None, y_out: torch.Tensor | None = None):
    """RMSNorm (with ``residual``: of x + residual, and ``residual`` is overwritten in place with bf16(x + residual),
    the stream the next layer adds to) fused with the static activation quantiser.
    Returns (xq or None, y or None): e4m3 codes [M, H] when ``input_scale`` is given, the bf16 result when
    ``want_bf16`` (or when there is no ``input_scale``)."""
    _require_cuda(x, weight, input_scale, residual)
    if x.dim() != 2 or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise ValueError("x must be a 2-D bfloat16 tensor and weight a bfloat16 vector")
    if x.stride(1) != 1:
        x = x.contiguous()
    m, h = x.shape
    if weight.numel() != h or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous vector of H elements")
    if residual is not None and (residual.shape != x.shape or residual.dtype != torch.bfloat16 or residual.stride(1) != 1):
        raise ValueError("residual must be a bfloat16 tensor of x's shape with contiguous rows (it is updated in place)")
    xq = y = None
    if input_scale is not None:
        xq = xq_out if xq_out is not None else torch.empty((m, h), dtype=torch.uint8, device=x.device)
    if want_bf16 or input_scale is None:
        y = y_out if y_out is not None else torch.empty((m, h), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().fp8lin_rmsnorm_quant(
            x.data_ptr(), x.stride(0), residual.data_ptr() if residual is not None else None,
            residual.stride(0) if residual is not None else 0, weight.data_ptr(), float(eps),
            input_scale.data_ptr() if input_scale is not None else None, xq.data_ptr() if xq is not None else None,
            y.data_ptr() if y is not None else None, y.stride(0) if y is not None else 0, m, h, _stream_ptr(x.device))
    _lib.raise_for(rc, "fp8lin_rmsnorm_quant")
    return xq, y


def quantize_activation(x: torch.Tensor, input_scale: torch.Tensor) -> torch.Tensor:
    """bf16 [M, K] -> e4m3 codes (uint8) with one static scale."""
    _require_cuda(x, input_scale)
    if x.dim() != 2 or x.dtype != torch.bfloat16:
        raise ValueError("x must be a 2-D bfloat16 tensor")
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    out = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().fp8lin_quantize_activation(x.data_ptr(), x.stride(0), input_scale.data_ptr(),
                                                    out.data_ptr(), m, k, _stream_ptr(x.device))
    _lib.raise_for(rc, "fp8lin_quantize_activation")
    return out


def launch_w8a8_scatter(x: torch.Tensor, w_packed: torch.Tensor, input_scale: torch.Tensor, weight_scale: torch.Tensor,
                        bias: torch.Tensor | None, dst_ptrs: list[int], ld_dst: int) -> None:
    """This rank's partial output of a row-parallel linear, stored by the GEMM epilogue into every
    destination (device pointers to bf16 [M, ld_dst] matrices, usually peer-mapped)."""
    x, n, k = _check_linear_args(x, w_packed, weight_scale, bias)
    m = x.shape[0]
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    with torch.cuda.device(x.device):
        ws = workspace(x.device, workspace_bytes(_lib.W8A8_STATIC, m, k, n))
        rc = _lib.load().fp8lin_w8a8_scatter(
            x.data_ptr(), x.stride(0), w_packed.data_ptr(), weight_scale.data_ptr(), input_scale.data_ptr(),
            bias.data_ptr() if bias is not None else None, len(dst_ptrs), arr, ld_dst, m, k, n,
            ws.data_ptr(), ws.numel(), _stream_ptr(x.device))
    _lib.raise_for(rc, "fp8lin_w8a8_scatter")


def launch_w8a8_reduce_scatter(x: torch.Tensor, w_packed: torch.Tensor, input_scale: torch.Tensor, weight_scale: torch.Tensor,
                               bias: torch.Tensor | None, dst_ptrs: list[int], ld_dst: int, band_rows: int) -> None:
    """This rank's partial output of a row-parallel linear, rows of band d stored only to ``dst_ptrs[d]``
    (device pointers to bf16 [band_rows, ld_dst] matrices: this rank's slot in rank d's buffer)."""
    x, n, k = _check_linear_args(x, w_packed, weight_scale, bias)
    m = x.shape[0]
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    with torch.cuda.device(x.device):
        ws = workspace(x.device, workspace_bytes(_lib.W8A8_STATIC, m, k, n))
        rc = _lib.load().fp8lin_w8a8_reduce_scatter(
            x.data_ptr(), x.stride(0), w_packed.data_ptr(), weight_scale.data_ptr(), input_scale.data_ptr(),
            bias.data_ptr() if bias is not None else None, len(dst_ptrs), arr, ld_dst, band_rows, m, k, n,
            ws.data_ptr(), ws.numel(), _stream_ptr(x.device))
    _lib.raise_for(rc, "fp8lin_w8a8_reduce_scatter")


def sum_slots_gather(slots_ptr: int, n_slots: int, slot_stride: int, ld_slot: int, dst_ptrs: list[int], ld_dst: int,
                     dst_row: int, m: int, n: int, device: torch.device) -> None:
    """Add ``n_slots`` bf16 [m, n] partials (``slot_stride`` elements apart) and store the sum at rows
    [dst_row, dst_row + m) of every matrix in ``dst_ptrs`` (the ranks' outputs; peers by NVLink stores)."""
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    with torch.cuda.device(device):
        rc = _lib.load().fp8lin_sum_slots_gather(slots_ptr, n_slots, slot_stride, ld_slot, len(dst_ptrs), arr, ld_dst,
                                                 dst_row, m, n, _stream_ptr(device))
    _lib.raise_for(rc, "fp8lin_sum_slots_gather")


def sum_slots(slots: torch.Tensor, m: int, n: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """slots: bf16 [n_slots, rows >= m, n] -> bf16 [m, n], slots added in order in fp32."""
    n_slots = slots.shape[0]
    y = out if out is not None else torch.empty((m, n), dtype=torch.bfloat16, device=slots.device)
    with torch.cuda.device(slots.device):
        rc = _lib.load().fp8lin_sum_slots(slots.data_ptr(), n_slots, slots.stride(0), slots.stride(1), y.data_ptr(),
                                          y.stride(0), m, n, _stream_ptr(slots.device))
    _lib.raise_for(rc, "fp8lin_sum_slots")
    return y


def interleave_gate_up(w_packed: torch.Tensor, weight_scale: torch.Tensor, bias: torch.Tensor | None, inter: int):
    """Reorder a packed merged gate_up weight ([2*inter, K]: gate rows, then up rows) so that its
    128-channel tile rows alternate gate / up, and permute scale and bias alike: the layout the
    fused MLP call takes.  A pure permutation of whole tile rows (no repacking)."""
    if inter % 128:
        raise ValueError(f"the intermediate size must be a multiple of 128 (got {inter})")
    t = inter // 128
    w = w_packed.view(2, t, -1).transpose(0, 1).contiguous().view(-1)
    s = weight_scale.view(2, t, 128).transpose(0, 1).contiguous().view(-1)
    b = bias.view(2, t, 128).transpose(0, 1).contiguous().view(-1) if bias is not None else None
    return w, s, b


def launch_mlp_w8a8(x: torch.Tensor, w_gate_up_il: torch.Tensor, gate_up_scale_il: torch.Tensor,
                    gate_up_input_scale: torch.Tensor, gate_up_bias_il: torch.Tensor | None, w_down: torch.Tensor,
                    down_scale: torch.Tensor, down_input_scale: torch.Tensor, down_bias: torch.Tensor | None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 ``down(silu(gate(x)) * up(x))`` with both projections W8A8-static; operands as produced by
    ``interleave_gate_up`` (gate_up) and ``pack_weight_nk`` / ``prepack_weight`` (down).  ``x`` is bfloat16
    [M, H], or uint8 [M, H] e4m3 codes already quantised with ``gate_up_input_scale`` (``rmsnorm_quant``)."""
    preq = x.dtype == torch.uint8
    if preq:
        if x.dim() != 2 or not x.is_contiguous() or not x.is_cuda:
            raise ValueError("pre-quantised activations must be a contiguous 2-D uint8 CUDA tensor")
        n2, h = gate_up_scale_il.numel(), x.shape[1]
        if h % 16 or w_gate_up_il.numel() != packed_bytes(h, n2):
            raise ValueError("the packed gate_up weight does not match the activations' width")
    else:
        x, n2, h = _check_linear_args(x, w_gate_up_il, gate_up_scale_il, gate_up_bias_il)
    inter = n2 // 2
    n = down_scale.numel()
    _require_cuda(w_down, down_scale, gate_up_input_scale, down_input_scale)
    if w_down.numel() != packed_bytes(inter, n):
        raise ValueError("w_down does not match the intermediate size of the gate_up weight")
    if down_bias is not None and (down_bias.dtype != torch.bfloat16 or down_bias.numel() != n):
        raise ValueError("down_bias must be bf16 [N]")
    m = x.shape[0]
    y = out if out is not None else torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        lib = _lib.load()
        ws = workspace(x.device, lib.fp8lin_mlp_workspace_bytes(m, h, inter, n))
        if preq:
            rc = lib.fp8lin_mlp_w8a8_preq(
                x.data_ptr(), w_gate_up_il.data_ptr(), gate_up_scale_il.data_ptr(), gate_up_input_scale.data_ptr(),
                gate_up_bias_il.data_ptr() if gate_up_bias_il is not None else None, w_down.data_ptr(), down_scale.data_ptr(),
                down_input_scale.data_ptr(), down_bias.data_ptr() if down_bias is not None else None, y.data_ptr(), y.stride(0),
                m, h, inter, n, ws.data_ptr(), ws.numel(), _stream_ptr(x.device))
            _lib.raise_for(rc, "fp8lin_mlp_w8a8_preq")
            return y
        rc = lib.fp8lin_mlp_w8a8(
            x.data_ptr(), x.stride(0), w_gate_up_il.data_ptr(), gate_up_scale_il.data_ptr(), gate_up_input_scale.data_ptr(),
            gate_up_bias_il.data_ptr() if gate_up_bias_il is not None else None, w_down.data_ptr(), down_scale.data_ptr(),
            down_input_scale.data_ptr(), down_bias.data_ptr() if down_bias is not None else None, y.data_ptr(), y.stride(0),
            m, h, inter, n, ws.data_ptr(), ws.numel(), _stream_ptr(x.device))
    _lib.raise_for(rc, "fp8lin_mlp_w8a8")
    return y
