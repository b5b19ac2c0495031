"""Host-side mirror of the reference's TW-Marlin interface, over the C ABI.

Function names, argument order and error behaviour follow the reference's
``warp_kernels::quantize`` module (crates/kernels/src/quantize.rs) so that a
test written against the reference reads the same here; tensors are torch CUDA
tensors standing in for ``GpuTensor<T>``.  torch only supplies device memory
and the current stream: every computation is a call into ``libtwmarlin.so``.

  gemm_tw_marlin_m1             quantize.rs:1301-1360
  gemm_tw_marlin_m1_from_buffer quantize.rs:1731-1782
  gemm_tw_marlin_m1_indirect    quantize_indirect.rs:228-253
  fuse_tw_marlin_n              quantize.rs:1018-1063
  quantize_f32_to_tw_marlin     quantize.rs:1171-1180
  cpu_quantize_tw_marlin        crates/loader/src/gemma_moe_q4.rs:218-254 (here: on the device)
  TWMarlinWeights               quantize.rs:1067-1165
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import GemmArgs, Plan, TwmError, check

BLOCK_SIZE = 32  # quantize.rs:25

_DTYPES = {torch.float32: _lib.TWM_F32, torch.float16: _lib.TWM_F16}


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise TwmError(_lib.TWM_EINVAL, "expected a CUDA tensor (there is no CPU path)")


def plan(m: int, n: int, k: int, group_size: int = BLOCK_SIZE, sm_count: int = 0,
         splits_override: int = 0, kernel_override: int = 0) -> Plan:
    """The tile / split-K decision for a shape (pure host arithmetic; replaces
    the heuristic of quantize.rs:1314-1325)."""
    out = Plan()
    check(_lib.lib().twm_plan(m, n, k, group_size, sm_count, splits_override, kernel_override, C.byref(out)),
          "twm_plan")
    return out


def workspace_bytes(m: int, n: int, k: int, group_size: int = BLOCK_SIZE) -> int:
    return int(_lib.lib().twm_workspace_bytes(m, n, k, group_size))


class Workspace:
    """Caller-owned split-K scratch.  Zeroed once here; the kernels hand its
    counters back at zero, so it is reusable launch after launch on one stream."""

    def __init__(self, nbytes: int, device: torch.device | str = "cuda"):
        self.nbytes = max(int(nbytes), 16)
        self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)

    @classmethod
    def for_shapes(cls, shapes: Sequence[Tuple[int, int, int, int]], device="cuda") -> "Workspace":
        """shapes: (M, N, K, group_size) of every GEMM that will share it."""
        return cls(max([workspace_bytes(*s) for s in shapes] + [16]), device)

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()


def gemm_tw_marlin(a: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, c: torch.Tensor,
                   m: int, n: int, k: int, *, group_size: int = BLOCK_SIZE,
                   workspace: Optional[Workspace] = None, stream: Optional[torch.cuda.Stream] = None,
                   flags: int = 0, splits_override: int = 0, kernel_override: int = 0,
                   packed_offsets: Optional[torch.Tensor] = None,
                   scales_offsets: Optional[torch.Tensor] = None, expert_idx: int = 0,
                   a_prologue: int = _lib.TWM_A_PLAIN, next_gemm: Optional[tuple] = None) -> None:
    """C[m,n] = A[m,k] x dequant(packed, scales); A and C are f32 or f16, row-major.

    The M > 1 form of ``gemm_tw_marlin_m1``; enqueue only, like the reference.  With
    ``a_prologue=TWM_A_SILU_MUL`` (m <= 32, f16) ``a`` is the [gate | up] output of the preceding GEMM
    (2k values) and the GEMM reads silu(gate) * up: fused_silu_mul (ops.rs:966-977) without its pass.
    ``next_gemm=(packed, scales, m, n, k, group_size)`` names the GEMM that follows on the stream (same
    dtypes and workspace): while this one drains, the head of that one's weights is pulled into L2."""
    _require_cuda(a, packed, scales, c)
    if a.dtype not in _DTYPES or c.dtype not in _DTYPES:
        raise TwmError(_lib.TWM_EINVAL, "gemm_tw_marlin: A and C must be float32 or float16")
    if packed.dtype != torch.uint8 or scales.dtype not in (torch.float16, torch.uint16, torch.int16):
        raise TwmError(_lib.TWM_EINVAL, "gemm_tw_marlin: packed must be uint8 and scales float16")
    a_cols = k if a_prologue == _lib.TWM_A_PLAIN else 2 * k
    if a.numel() < m * a_cols or c.numel() < m * n:
        raise TwmError(_lib.TWM_EINVAL, "gemm_tw_marlin: A or C smaller than the stated shape")
    if packed_offsets is None:
        if packed.numel() < (k // 32) * n * 16 or scales.numel() < (k // group_size) * n:
            raise TwmError(_lib.TWM_EINVAL, "gemm_tw_marlin: packed or scales smaller than the stated shape")
    lda = a.stride(0) if a.dim() == 2 else a_cols
    ldc = c.stride(0) if c.dim() == 2 else n
    args = GemmArgs(
        M=m, N=n, K=k, group_size=group_size,
        a_dtype=_DTYPES[a.dtype], c_dtype=_DTYPES[c.dtype],
        a=a.data_ptr(), lda=lda, packed=packed.data_ptr(), scales=scales.data_ptr(),
        c=c.data_ptr(), ldc=ldc,
        workspace=workspace.ptr if workspace is not None else None,
        workspace_bytes=workspace.nbytes if workspace is not None else 0,
        splits_override=splits_override, kernel_override=kernel_override, flags=flags,
        packed_offsets=packed_offsets.data_ptr() if packed_offsets is not None else None,
        scales_offsets=scales_offsets.data_ptr() if scales_offsets is not None else None,
        expert_idx=expert_idx, a_prologue=a_prologue,
    )
    if next_gemm is not None:
        np_, ns_, nm, nn, nk, ng = next_gemm
        nxt = GemmArgs(M=nm, N=nn, K=nk, group_size=ng, a_dtype=args.a_dtype, c_dtype=args.c_dtype,
                       packed=np_.data_ptr(), scales=ns_.data_ptr(), workspace=args.workspace,
                       workspace_bytes=args.workspace_bytes)
        args.next = C.addressof(nxt)          # read during the call below only
    check(_lib.lib().twm_gemm_w4a16(C.byref(args), _stream_ptr(stream)), "twm_gemm_w4a16")


def gemm_tw_marlin_m1(a: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, c: torch.Tensor,
                      n: int, k: int, **kw) -> None:
    """Drop-in for ``gemm_tw_marlin_m1(cache, device, a, packed, scales, c, n, k)``
    (quantize.rs:1301-1310).  The kernel cache and device arguments have no
    counterpart: kernels are compiled ahead of time and the device is the
    tensors' device."""
    if k % BLOCK_SIZE != 0:
        raise TwmError(_lib.TWM_EINVAL, "gemm_tw_marlin_m1: k % 32 != 0")   # the reference asserts (quantize.rs:1311)
    gemm_tw_marlin(a, packed, scales, c, 1, n, k, **kw)


def gemm_tw_marlin_m1_from_buffer(a, packed_buf: torch.Tensor, packed_offset: int, scales_buf: torch.Tensor,
                                  scales_offset: int, c, n: int, k: int, **kw) -> None:
    """``gemm_tw_marlin_m1`` on a sub-range of two big buffers (quantize.rs:1731-1741):
    packed_offset in bytes, scales_offset in elements, both applied on the host."""
    g = kw.get("group_size", BLOCK_SIZE)
    pv = packed_buf.view(-1)[packed_offset:packed_offset + (k // 32) * n * 16]
    sv = scales_buf.view(-1)[scales_offset:scales_offset + (k // g) * n]
    gemm_tw_marlin_m1(a, pv, sv, c, n, k, **kw)


def gemm_tw_marlin_m1_indirect(a, packed_buf, packed_offsets: torch.Tensor, scales_buf,
                               scales_offsets: torch.Tensor, expert_idx: int, c, n: int, k: int, **kw) -> None:
    """Expert-indexed form (quantize_indirect.rs:228-237): the kernel itself reads
    ``packed_offsets[expert_idx]`` (bytes) and ``scales_offsets[expert_idx]`` (elements)."""
    gemm_tw_marlin(a, packed_buf, scales_buf, c, 1, n, k, packed_offsets=packed_offsets,
                   scales_offsets=scales_offsets, expert_idx=expert_idx, **kw)


def quantize_f32_to_tw_marlin(weights: torch.Tensor, k: int, n: int, group_size: int = BLOCK_SIZE,
                              *, w_is_nk: bool = False, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """F32 weights -> (packed u8 [k/32, n, 16], scales f16 [k/group, n]).

    ``weights`` is [K,N] row-major as for the reference's function of this name
    (quantize.rs:1171-1177), or [N,K] with ``w_is_nk`` as ``cpu_quantize_tw_marlin``
    takes it (gemma_moe_q4.rs:214)."""
    _require_cuda(weights)
    if weights.dtype != torch.float32 or weights.numel() != k * n or not weights.is_contiguous():
        raise TwmError(_lib.TWM_EINVAL, "quantize_f32_to_tw_marlin: need contiguous float32 of k*n elements")
    packed = torch.empty((k // 32, n, 16), dtype=torch.uint8, device=weights.device)
    scales = torch.empty((k // group_size, n), dtype=torch.float16, device=weights.device)
    check(_lib.lib().twm_quantize_pack(weights.data_ptr(), int(w_is_nk), k, n, group_size, packed.data_ptr(),
                                       scales.data_ptr(), _stream_ptr(stream)), "twm_quantize_pack")
    return packed, scales


def reorder_to_tw_marlin(col_major_q4: torch.Tensor, k: int, n: int, *, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Column-major Q4_0 blocks (20 bytes each: f32 scale + 16 nibble bytes, block (col, g) at
    (col * k/32 + g) * 20) -> (packed u8 [k/32, n, 16], scales f16 [k/32, n]), on the device
    (reorder_to_tw_marlin, quantize.rs:912-917; the reference does this on the host)."""
    _require_cuda(col_major_q4)
    if col_major_q4.dtype != torch.uint8 or col_major_q4.numel() != (k // 32) * n * 20 or not col_major_q4.is_contiguous():
        raise TwmError(_lib.TWM_EINVAL, "reorder_to_tw_marlin: need contiguous uint8 of (k/32)*n*20 bytes")
    packed = torch.empty((k // 32, n, 16), dtype=torch.uint8, device=col_major_q4.device)
    scales = torch.empty((k // 32, n), dtype=torch.float16, device=col_major_q4.device)
    check(_lib.lib().twm_reorder_to_tw_marlin(col_major_q4.data_ptr(), k, n, packed.data_ptr(), scales.data_ptr(),
                                              _stream_ptr(stream)), "twm_reorder_to_tw_marlin")
    return packed, scales


def cpu_quantize_tw_marlin(data_nk: torch.Tensor, k: int, n: int, group_size: int = BLOCK_SIZE):
    """Same tensors as the reference's CPU quantiser of this name
    (gemma_moe_q4.rs:218-254), produced on the device from [N,K] input."""
    return quantize_f32_to_tw_marlin(data_nk, k, n, group_size, w_is_nk=True)


def dequant_tw_marlin(packed: torch.Tensor, scales: torch.Tensor, k: int, n: int,
                      group_size: int = BLOCK_SIZE, dtype: torch.dtype = torch.float32, *, stream=None) -> torch.Tensor:
    """Dense [K,N] matrix w = f32(scale) * (nibble - 8); f32 is exact, f16 rounds
    to nearest even (dequant_q4_to_f16, quantize.rs:580-618)."""
    _require_cuda(packed, scales)
    out = torch.empty((k, n), dtype=dtype, device=packed.device)
    check(_lib.lib().twm_dequant(packed.data_ptr(), scales.data_ptr(), out.data_ptr(), _DTYPES[dtype], k, n,
                                 group_size, _stream_ptr(stream)), "twm_dequant")
    return out


def fuse_tw_marlin_n(matrices: Sequence[Tuple[torch.Tensor, torch.Tensor]], k: int, ns: Sequence[int],
                     group_size: int = BLOCK_SIZE, *, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Concatenate along N, block row by block row (quantize.rs:1018-1063), on
    the device instead of through the host."""
    cnt = len(matrices)
    if cnt == 0 or cnt != len(ns):
        raise TwmError(_lib.TWM_EINVAL, "fuse_tw_marlin_n: matrices and ns differ in length")
    for (p, s), n_i in zip(matrices, ns):
        _require_cuda(p, s)
        if p.numel() != (k // 32) * n_i * 16 or s.numel() != (k // group_size) * n_i:
            raise TwmError(_lib.TWM_EINVAL, "fuse_tw_marlin_n: a matrix does not match k and its n")
    total = int(sum(ns))
    dev = matrices[0][0].device
    packed = torch.empty((k // 32, total, 16), dtype=torch.uint8, device=dev)
    scales = torch.empty((k // group_size, total), dtype=torch.float16, device=dev)
    pp = (C.c_void_p * cnt)(*[p.data_ptr() for p, _ in matrices])
    sp = (C.c_void_p * cnt)(*[s.data_ptr() for _, s in matrices])
    nn = (C.c_int * cnt)(*[int(x) for x in ns])
    check(_lib.lib().twm_fuse_n(pp, sp, nn, cnt, k, group_size, packed.data_ptr(), scales.data_ptr(),
                                _stream_ptr(stream)), "twm_fuse_n")
    return packed, scales


def slice_tw_marlin_n(packed: torch.Tensor, scales: torch.Tensor, k: int, n: int, n0: int, n_len: int,
                      group_size: int = BLOCK_SIZE, *, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Columns [n0, n0+n_len) as their own TW-Marlin matrix (column shard)."""
    _require_cuda(packed, scales)
    p = torch.empty((k // 32, n_len, 16), dtype=torch.uint8, device=packed.device)
    s = torch.empty((k // group_size, n_len), dtype=torch.float16, device=packed.device)
    check(_lib.lib().twm_slice_n(packed.data_ptr(), scales.data_ptr(), k, n, group_size, n0, n_len, p.data_ptr(),
                                 s.data_ptr(), _stream_ptr(stream)), "twm_slice_n")
    return p, s


def slice_tw_marlin_k(packed: torch.Tensor, scales: torch.Tensor, k: int, n: int, k0: int, k_len: int,
                      group_size: int = BLOCK_SIZE) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows [k0, k0+k_len) (row shard): contiguous, so these are views."""
    po, so = C.c_size_t(), C.c_size_t()
    check(_lib.lib().twm_slice_k_offsets(k, n, group_size, k0, k_len, C.byref(po), C.byref(so)),
          "twm_slice_k_offsets")
    p = packed.view(-1)[po.value:po.value + (k_len // 32) * n * 16].view(k_len // 32, n, 16)
    s = scales.view(-1)[so.value:so.value + (k_len // group_size) * n].view(k_len // group_size, n)
    return p, s


def moe_workspace_bytes(top_k: int, n: int, k: int, group_size: int = BLOCK_SIZE) -> int:
    return int(_lib.lib().twm_moe_workspace_bytes(top_k, n, k, group_size))


def _moe_args(a, a_slot_stride, a_prologue, packed_buf, scales_buf, topk_ids, topk_weights, c, c_slot_stride,
              packed_bytes_per_expert, scales_per_expert, n, k, top_k, group_size, workspace, flags):
    _require_cuda(a, packed_buf, scales_buf, topk_ids, c)
    if a.dtype != torch.float16 or c.dtype not in _DTYPES or topk_ids.dtype != torch.float32:
        raise TwmError(_lib.TWM_EINVAL, "expert GEMV: activations float16, output float16/float32, expert ids float32")
    return _lib.MoeArgs(top_k=top_k, N=n, K=k, group_size=group_size, a=a.data_ptr(), a_slot_stride=a_slot_stride,
                        a_prologue=a_prologue, packed_base=packed_buf.data_ptr(), scales_base=scales_buf.data_ptr(),
                        packed_bytes_per_expert=packed_bytes_per_expert, scales_per_expert=scales_per_expert,
                        topk_ids=topk_ids.data_ptr(),
                        topk_weights=topk_weights.data_ptr() if topk_weights is not None else None,
                        c=c.data_ptr(), c_dtype=_DTYPES[c.dtype], c_slot_stride=c_slot_stride,
                        workspace=workspace.ptr if workspace is not None else None,
                        workspace_bytes=workspace.nbytes if workspace is not None else 0, flags=flags)


def batched_marlin_gate_up(input: torch.Tensor, packed_buf: torch.Tensor, scales_buf: torch.Tensor, topk_ids: torch.Tensor,
                           output: torch.Tensor, packed_bytes_per_expert: int, scales_per_expert: int, n: int, k: int,
                           top_k: int, *, group_size: int = BLOCK_SIZE, workspace: Optional[Workspace] = None,
                           stream=None, flags: int = 0) -> None:
    """All top_k experts' gate+up GEMVs in one launch (batched_marlin_gate_up,
    moe_batched_marlin.rs:155-185): output[e, :] = input x W[topk_ids[e]].  `input` is one f16 row of
    k values, `output` is [top_k, n]."""
    args = _moe_args(input, 0, _lib.TWM_A_PLAIN, packed_buf, scales_buf, topk_ids, None, output, n,
                     packed_bytes_per_expert, scales_per_expert, n, k, top_k, group_size, workspace, flags)
    check(_lib.lib().twm_moe_gate_up(C.byref(args), _stream_ptr(stream)), "twm_moe_gate_up")


def batched_marlin_down_axpy(gate_up_all: torch.Tensor, packed_buf: torch.Tensor, scales_buf: torch.Tensor,
                             topk_ids: torch.Tensor, topk_weights: torch.Tensor, acc: torch.Tensor,
                             packed_bytes_per_expert: int, scales_per_expert: int, n: int, k: int, top_k: int, *,
                             activation: str = "geglu", group_size: int = BLOCK_SIZE,
                             workspace: Optional[Workspace] = None, stream=None, flags: int = 0) -> None:
    """All top_k experts' down GEMVs and the router-weighted sum in one launch
    (batched_marlin_split_geglu + batched_marlin_down_axpy, moe_batched_marlin.rs:187-233).
    gate_up_all is the gate+up output [top_k, 2k] (f16): the kernel reads gelu_tanh(gate) * up
    ("geglu"), silu(gate) * up ("swiglu"), or with activation="none" a [top_k, k] tensor as it is.
    acc[n] = (acc[n] with TWM_FLAG_ACCUMULATE) + sum over slots in slot order."""
    pro = {"geglu": _lib.TWM_A_GEGLU, "swiglu": _lib.TWM_A_SILU_MUL, "none": _lib.TWM_A_PLAIN}[activation]
    stride = k if pro == _lib.TWM_A_PLAIN else 2 * k
    if topk_weights.dtype != torch.float32:
        raise TwmError(_lib.TWM_EINVAL, "batched_marlin_down_axpy: router weights must be float32")
    args = _moe_args(gate_up_all, stride, pro, packed_buf, scales_buf, topk_ids, topk_weights, acc, 0,
                     packed_bytes_per_expert, scales_per_expert, n, k, top_k, group_size, workspace, flags)
    check(_lib.lib().twm_moe_down_axpy(C.byref(args), _stream_ptr(stream)), "twm_moe_down_axpy")


class GemmChain:
    """A list of GEMMs that run, in order, as ONE persistent launch (``twm_chain_*``).

    The reference enqueues the four GEMMs of a layer one kernel at a time
    (generate.rs:2149-2206); a chain keeps the weight stream going across the boundaries
    between them.  ``add`` takes the arguments of ``gemm_tw_marlin``; ``build`` is the set-up
    call (allocates); ``launch`` only enqueues."""

    def __init__(self):
        self._ops = []
        self._keep = []            # the tensors the device-side table points at
        self._handle = None

    def add(self, a: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, c: torch.Tensor, m: int, n: int, k: int,
            *, group_size: int = BLOCK_SIZE, flags: int = 0, silu_mul: bool = False) -> "GemmChain":
        """C[m,n] (+)= A x dequant(packed, scales).  With ``silu_mul`` A is the fused gate+up
        output [m, 2k] and the GEMM reads silu(gate) * up."""
        if self._handle is not None:
            raise TwmError(_lib.TWM_EINVAL, "GemmChain.add after build")
        _require_cuda(a, packed, scales, c)
        if a.dtype != torch.float16 or c.dtype not in _DTYPES:
            raise TwmError(_lib.TWM_EINVAL, "GemmChain.add: A must be float16, C float16 or float32")
        need_a = m * k * (2 if silu_mul else 1)
        if a.numel() < need_a or c.numel() < m * n:
            raise TwmError(_lib.TWM_EINVAL, "GemmChain.add: A or C smaller than the stated shape")
        if packed.numel() < (k // 32) * n * 16 or scales.numel() < (k // group_size) * n:
            raise TwmError(_lib.TWM_EINVAL, "GemmChain.add: packed or scales smaller than the stated shape")
        lda = a.stride(0) if a.dim() == 2 else k * (2 if silu_mul else 1)
        ldc = c.stride(0) if c.dim() == 2 else n
        op = _lib.ChainOp()
        op.gemm = GemmArgs(M=m, N=n, K=k, group_size=group_size, a_dtype=_lib.TWM_F16, c_dtype=_DTYPES[c.dtype],
                           a=a.data_ptr(), lda=lda, packed=packed.data_ptr(), scales=scales.data_ptr(),
                           c=c.data_ptr(), ldc=ldc, flags=flags)
        op.gemm.a_prologue = _lib.TWM_A_SILU_MUL if silu_mul else _lib.TWM_A_PLAIN
        self._ops.append(op)
        self._keep.append((a, packed, scales, c))
        return self

    def build(self) -> "GemmChain":
        n = len(self._ops)
        arr = (_lib.ChainOp * n)(*self._ops)
        h = C.c_void_p()
        check(_lib.lib().twm_chain_create(arr, n, C.byref(h)), "twm_chain_create")
        self._handle = h
        return self

    @property
    def info(self) -> "_lib.ChainInfo":
        out = _lib.ChainInfo()
        check(_lib.lib().twm_chain_info(self._handle, C.byref(out)), "twm_chain_info")
        return out

    def launch(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        if self._handle is None:
            self.build()
        check(_lib.lib().twm_chain_launch(self._handle, _stream_ptr(stream)), "twm_chain_launch")

    def close(self) -> None:
        if self._handle is not None:
            _lib.lib().twm_chain_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def chain_partition(n_tiles: int, nkb: int, grid: int, rank: int):
    """The pieces (tile, blk0, blk1, slot, n_pieces) a chain gives `rank` of `grid` for one GEMM."""
    cap = 64
    while True:
        buf = (C.c_int * (5 * cap))()
        n = C.c_int(0)
        check(_lib.lib().twm_chain_partition(n_tiles, nkb, grid, rank, cap, buf, C.byref(n)), "twm_chain_partition")
        if n.value <= cap:
            return [tuple(buf[5 * i:5 * i + 5]) for i in range(n.value)]
        cap = n.value


def device_error(stream=None) -> int:
    """Read and clear the device-side error word (synchronises the stream)."""
    w = C.c_uint(0)
    st = _lib.lib().twm_device_error(_stream_ptr(stream), C.byref(w))
    if st not in (_lib.TWM_OK, _lib.TWM_ETIMEOUT):
        check(st, "twm_device_error")
    return int(w.value)


@dataclass
class TWMarlinWeights:
    """One transformer layer in TW-Marlin form (quantize.rs:1067-1086): norms,
    seven projections as (packed, scales), optional q/k/v bias, optional fused
    QKV and gate+up."""
    hidden: int
    kv_dim: int
    ffn: int
    group_size: int
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    wq: Tuple[torch.Tensor, torch.Tensor]
    wk: Tuple[torch.Tensor, torch.Tensor]
    wv: Tuple[torch.Tensor, torch.Tensor]
    wo: Tuple[torch.Tensor, torch.Tensor]
    w_gate: Tuple[torch.Tensor, torch.Tensor]
    w_up: Tuple[torch.Tensor, torch.Tensor]
    w_down: Tuple[torch.Tensor, torch.Tensor]
    bq: Optional[torch.Tensor] = None
    bk: Optional[torch.Tensor] = None
    bv: Optional[torch.Tensor] = None
    wqkv: Optional[Tuple[torch.Tensor, torch.Tensor]] = field(default=None)
    wgu: Optional[Tuple[torch.Tensor, torch.Tensor]] = field(default=None)

    @classmethod
    def from_quantized(cls, qw: dict, hidden: int, kv_dim: int, ffn: int, fuse: bool = False) -> "TWMarlinWeights":
        """From a layer held as column-major Q4_0 blocks (TWMarlinWeights::from_quantized,
        quantize.rs:1090-1134).  `qw` maps the reference's field names (wq, wk, wv, wo, w_gate, w_up,
        w_down: uint8 block tensors; attn_norm, ffn_norm: f32; optional bq, bk, bv) to tensors.  Scale
        group 32, as the blocks carry it."""
        def r(name, k, n):
            return reorder_to_tw_marlin(qw[name], k, n)
        out = cls(hidden=hidden, kv_dim=kv_dim, ffn=ffn, group_size=32, attn_norm=qw["attn_norm"].clone(),
                  ffn_norm=qw["ffn_norm"].clone(), wq=r("wq", hidden, hidden), wk=r("wk", hidden, kv_dim),
                  wv=r("wv", hidden, kv_dim), wo=r("wo", hidden, hidden), w_gate=r("w_gate", hidden, ffn),
                  w_up=r("w_up", hidden, ffn), w_down=r("w_down", ffn, hidden),
                  bq=qw.get("bq"), bk=qw.get("bk"), bv=qw.get("bv"))
        if fuse:
            out.fuse_projections()
        return out

    def fuse_projections(self) -> None:
        """Build the fused QKV and gate+up matrices (quantize.rs:1138-1165)."""
        g = self.group_size
        self.wqkv = fuse_tw_marlin_n([self.wq, self.wk, self.wv], self.hidden,
                                     [self.hidden, self.kv_dim, self.kv_dim], g)
        self.wgu = fuse_tw_marlin_n([self.w_gate, self.w_up], self.hidden, [self.ffn, self.ffn], g)
