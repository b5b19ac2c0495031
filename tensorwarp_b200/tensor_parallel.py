"""Tensor-parallel decode layer stack for one multi-GPU box, one process per GPU.

The reference has no device-side collective: its multi-GPU helper gathers on the host
(crates/kernels/src/multi_gpu.rs:128-366, "Peer-to-peer or NCCL would be faster" :327-328).  This
module is the tensor-parallel layer the benchmark configuration adds for the 70B-shaped stack:

* QKV and gate+up are column-sharded: rank r owns q heads [r*H/tp, (r+1)*H/tp), kv heads likewise,
  and the matching slices [gate_r | up_r], so RoPE, attention and SwiGLU stay local
  (a column shard of a TW-Marlin tensor is a column slice of every block row, the inverse of
  fuse_tw_marlin_n, quantize.rs:1038-1055);
* o and down are row-sharded along K at multiples of the scale group (a contiguous range of block
  rows); their [M, hidden] FP32 partial outputs are summed over ranks with one all-reduce each
  (NCCL over NVLink when run under torch.distributed, any callable otherwise) and join the FP32
  residual stream in the next fused add + RMSNorm.

The shard arithmetic is pure Python so that it can be tested without a GPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch

from . import _lib
from . import quantize as q
from ._lib import check
from .generate import TransformerConfig

LLAMA3_70B = TransformerConfig(hidden=8192, num_heads=64, num_kv_heads=8, head_dim=128, ffn=28672, vocab=128256,
                               layers=80, rope_theta=5e5, eps=1e-5, max_seq=8192, group_size=128, qkv_bias=False)


@dataclass(frozen=True)
class ShardSpec:
    """What rank `rank` of `tp` owns."""
    tp: int
    rank: int
    q_heads: Tuple[int, int]        # [first, last) query heads
    kv_heads: Tuple[int, int]
    ffn: Tuple[int, int]            # [first, last) columns of gate (and of up)
    q_cols: Tuple[int, int]         # columns of the q projection = rows (K range) of o
    kv_cols: Tuple[int, int]
    n_qkv: int                      # width of the local fused [q | k | v]
    n_gu: int                       # width of the local fused [gate | up]


def shard_spec(cfg: TransformerConfig, tp: int, rank: int) -> ShardSpec:
    if tp < 1 or not (0 <= rank < tp):
        raise ValueError("rank outside the group")
    if cfg.num_heads % tp or cfg.num_kv_heads % tp or cfg.ffn % tp:
        raise ValueError("heads, kv heads and ffn must divide by the tensor-parallel degree")
    if (cfg.ffn // tp) % cfg.group_size or (cfg.num_heads // tp * cfg.head_dim) % cfg.group_size:
        raise ValueError("row shards of o and down must hold whole scale groups")
    hq, hk, f = cfg.num_heads // tp, cfg.num_kv_heads // tp, cfg.ffn // tp
    qh = (rank * hq, (rank + 1) * hq)
    kh = (rank * hk, (rank + 1) * hk)
    return ShardSpec(tp=tp, rank=rank, q_heads=qh, kv_heads=kh, ffn=(rank * f, (rank + 1) * f),
                     q_cols=(qh[0] * cfg.head_dim, qh[1] * cfg.head_dim),
                     kv_cols=(kh[0] * cfg.head_dim, kh[1] * cfg.head_dim),
                     n_qkv=(hq + 2 * hk) * cfg.head_dim, n_gu=2 * f)


@dataclass
class TPLayerWeights:
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    wqkv: Tuple[torch.Tensor, torch.Tensor]        # [hidden, n_qkv] local columns
    wo: Tuple[torch.Tensor, torch.Tensor]          # [q_dim/tp, hidden] local rows
    wgu: Tuple[torch.Tensor, torch.Tensor]         # [hidden, n_gu]
    w_down: Tuple[torch.Tensor, torch.Tensor]      # [ffn/tp, hidden]
    bqkv: Optional[torch.Tensor] = None


def shard_layer(cfg: TransformerConfig, spec: ShardSpec, wq, wk, wv, wo, w_gate, w_up, w_down, attn_norm, ffn_norm,
                bias=None) -> TPLayerWeights:
    """Cut one layer's full TW-Marlin tensors down to a rank's share (twm_slice_n / row views / twm_fuse_n)."""
    g, h = cfg.group_size, cfg.hidden

    def cols(w, k, n, c0, c1):
        return q.slice_tw_marlin_n(w[0], w[1], k, n, c0, c1 - c0, g)

    q_s = cols(wq, h, cfg.q_dim, *spec.q_cols)
    k_s = cols(wk, h, cfg.kv_dim, *spec.kv_cols)
    v_s = cols(wv, h, cfg.kv_dim, *spec.kv_cols)
    nq, nk = spec.q_cols[1] - spec.q_cols[0], spec.kv_cols[1] - spec.kv_cols[0]
    wqkv = q.fuse_tw_marlin_n([q_s, k_s, v_s], h, [nq, nk, nk], g)
    g_s = cols(w_gate, h, cfg.ffn, *spec.ffn)
    u_s = cols(w_up, h, cfg.ffn, *spec.ffn)
    nf = spec.ffn[1] - spec.ffn[0]
    wgu = q.fuse_tw_marlin_n([g_s, u_s], h, [nf, nf], g)
    wo_s = q.slice_tw_marlin_k(wo[0], wo[1], cfg.q_dim, h, spec.q_cols[0], nq, g)
    wd_s = q.slice_tw_marlin_k(w_down[0], w_down[1], cfg.ffn, h, spec.ffn[0], nf, g)
    b = None
    if bias is not None:
        b = torch.cat([bias[spec.q_cols[0]:spec.q_cols[1]],
                       bias[cfg.q_dim + spec.kv_cols[0]:cfg.q_dim + spec.kv_cols[1]],
                       bias[cfg.q_dim + cfg.kv_dim + spec.kv_cols[0]:cfg.q_dim + cfg.kv_dim + spec.kv_cols[1]]]).contiguous()
    return TPLayerWeights(attn_norm=attn_norm, ffn_norm=ffn_norm, wqkv=wqkv, wo=(wo_s[0].contiguous(), wo_s[1].contiguous()),
                          wgu=wgu, w_down=(wd_s[0].contiguous(), wd_s[1].contiguous()), bqkv=b)


def random_shard_layer(cfg: TransformerConfig, spec: ShardSpec, layer: int, device, seed: int = 0) -> TPLayerWeights:
    """A rank's share generated directly (the benchmark's random-init weights: no rank ever holds a
    full 70B-shaped matrix)."""
    g, h = cfg.group_size, cfg.hidden
    nq = spec.q_cols[1] - spec.q_cols[0]
    nf = spec.ffn[1] - spec.ffn[0]

    def rnd(k, n, pid):
        gen = torch.Generator(device=device).manual_seed(seed + 1000 * layer + 10 * pid + 100000 * (spec.rank + 1))
        w = torch.randn((k, n), generator=gen, device=device, dtype=torch.float32) * 0.02
        out = q.quantize_f32_to_tw_marlin(w, k, n, g)
        del w
        return out

    ones = torch.ones(h, device=device)
    return TPLayerWeights(attn_norm=ones, ffn_norm=ones, wqkv=rnd(h, spec.n_qkv, 0), wo=rnd(nq, h, 3),
                          wgu=rnd(h, spec.n_gu, 4), w_down=rnd(nf, h, 6))


class PeerComm:
    """One rank's view of the group's receive buffers for the one-shot all-reduce that the
    row-parallel GEMMs push into (``twm_comm``).  Between processes the buffers are shared through
    CUDA IPC; inside one process (tests on a single GPU) they are plain allocations."""

    def __init__(self, n_ranks: int, rank: int, slot_elems: int, bases: List[int], owned: Optional[int] = None,
                 opened: Optional[List[int]] = None, wait_ms: float = 0.0):
        lib = _lib.lib()
        self.n_ranks, self.rank, self.slot_elems = n_ranks, rank, slot_elems
        self._owned, self._opened = owned, opened or []
        # wait_ms: how long the consumer kernel waits for the peers' partials (0 = the library's two seconds)
        self.struct = _lib.Comm(n_ranks=n_ranks, rank=rank, slot_elems=slot_elems, wait_ns=int(wait_ms * 1e6))
        for s_, base in enumerate(bases):
            d, f, st = C.c_void_p(), C.c_void_p(), C.c_void_p()
            check(lib.twm_comm_layout(C.c_void_p(base), n_ranks, slot_elems, C.byref(d), C.byref(f), C.byref(st)),
                  "twm_comm_layout")
            self.struct.data[s_] = d.value
            self.struct.flags[s_] = f.value
            if s_ == rank:
                self.struct.state = st.value

    @property
    def ptr(self) -> int:
        return C.addressof(self.struct)

    @staticmethod
    def _alloc(nbytes: int) -> int:
        p = C.c_void_p()
        check(_lib.lib().twm_ipc_alloc(nbytes, C.byref(p)), "twm_ipc_alloc")
        return p.value

    @classmethod
    def local_group(cls, n_ranks: int, slot_elems: int, wait_ms: float = 0.0) -> List["PeerComm"]:
        """All ranks in this process, on the current device (single-GPU emulation)."""
        nbytes = _lib.lib().twm_comm_bytes(n_ranks, slot_elems)
        bases = [cls._alloc(nbytes) for _ in range(n_ranks)]
        return [cls(n_ranks, r, slot_elems, bases, owned=bases[r], wait_ms=wait_ms) for r in range(n_ranks)]

    @classmethod
    def distributed(cls, slot_elems: int, wait_ms: float = 0.0) -> "PeerComm":
        """One rank per process under torch.distributed: allocate, exchange IPC handles, map the peers."""
        import torch.distributed as dist
        lib = _lib.lib()
        n, r = dist.get_world_size(), dist.get_rank()
        mine = cls._alloc(lib.twm_comm_bytes(n, slot_elems))
        hbuf = C.create_string_buffer(64)
        check(lib.twm_ipc_get_handle(C.c_void_p(mine), hbuf), "twm_ipc_get_handle")
        handles: List[Optional[bytes]] = [None] * n
        dist.all_gather_object(handles, bytes(hbuf.raw))
        bases, opened = [], []
        for s_ in range(n):
            if s_ == r:
                bases.append(mine)
            else:
                p = C.c_void_p()
                check(lib.twm_ipc_open(C.create_string_buffer(handles[s_], 64), C.byref(p)), "twm_ipc_open")
                bases.append(p.value)
                opened.append(p.value)
        dist.barrier()
        return cls(n, r, slot_elems, bases, owned=mine, opened=opened, wait_ms=wait_ms)

    def close(self) -> None:
        lib = _lib.lib()
        for p in self._opened:
            lib.twm_ipc_close(C.c_void_p(p))
        self._opened = []
        if self._owned is not None:
            lib.twm_ipc_free(C.c_void_p(self._owned))
            self._owned = None


class TPDecodeStack:
    """One rank's decode layer stack for `rows` sequences decoding in lock step (configs[4]: the
    layer stack only, no embedding or LM head)."""

    def __init__(self, cfg: TransformerConfig, spec: ShardSpec, layers: List[TPLayerWeights], rows: int, device,
                 all_reduce: Callable[[torch.Tensor], None], use_pdl: bool = True, comm: Optional[PeerComm] = None):
        self.cfg, self.spec, self.layers, self.rows = cfg, spec, layers, rows
        self.device = torch.device(device)
        self.all_reduce = all_reduce
        # With `comm` (and at most 64 rows, one GEMM launch) the row-parallel GEMMs push their FP32 result
        # straight into every rank's receive buffer and the following add + RMSNorm kernel takes the
        # sum: no collective call, no extra launch.  Otherwise `all_reduce` (NCCL) runs on `part`.
        self.comm = comm if (comm is not None and rows <= 64) else None
        if self.comm is not None and self.comm.slot_elems < rows * cfg.hidden:
            raise ValueError("comm slots are smaller than rows * hidden")
        self.flags = _lib.TWM_FLAG_PDL if use_pdl else 0
        f16, f32, i32 = torch.float16, torch.float32, torch.int32
        dev, m, h, hd = self.device, rows, cfg.hidden, cfg.head_dim
        hq = spec.q_heads[1] - spec.q_heads[0]
        hk = spec.kv_heads[1] - spec.kv_heads[0]
        self.hq, self.hk = hq, hk
        self.x = torch.zeros((m, h), dtype=f32, device=dev)
        self.part = torch.zeros((m, h), dtype=f32, device=dev)          # row-parallel partial, all-reduced in place
        self.normed = torch.zeros((m, h), dtype=f16, device=dev)
        self.qkv = torch.zeros((m, spec.n_qkv), dtype=f16, device=dev)
        self.rope_table = torch.zeros(hd, dtype=torch.float32, device=dev)       # cos | sin of the step's position
        self.attn = torch.zeros((m, hq * hd), dtype=f16, device=dev)
        self.gate_up = torch.zeros((m, spec.n_gu), dtype=f16, device=dev)
        self.act = torch.zeros((m, spec.n_gu // 2), dtype=f16, device=dev)
        self.pos = torch.zeros(1, dtype=i32, device=dev)
        self.cache_len = torch.zeros(1, dtype=i32, device=dev)
        self.k_cache = [torch.zeros((m, cfg.max_seq, hk * hd), dtype=f16, device=dev) for _ in layers]
        self.v_cache = [torch.zeros((m, cfg.max_seq, hk * hd), dtype=f16, device=dev) for _ in layers]
        lib = _lib.lib()
        self.attn_scratch = torch.zeros(lib.twm_attn_scratch_bytes(m, hq, hd, cfg.max_seq), dtype=torch.uint8, device=dev)
        g = cfg.group_size
        shapes = [(m, spec.n_qkv, h, g), (m, h, hq * hd, g), (m, spec.n_gu, h, g), (m, h, spec.n_gu // 2, g)]
        self.workspace = q.Workspace.for_shapes(shapes, dev)
        self.pending_add = False
        self.launches = 0

    def prefill_random_kv(self, length: int, seed: int = 2) -> None:
        gen = torch.Generator(device=self.device).manual_seed(seed + 17 * self.spec.rank)
        for kc, vc in zip(self.k_cache, self.v_cache):
            kc[:, :length] = torch.randn(kc[:, :length].shape, generator=gen, device=self.device).half()
            vc[:, :length] = torch.randn(vc[:, :length].shape, generator=gen, device=self.device).half()
        self.pos.fill_(length)
        self.cache_len.fill_(length + 1)

    def _gemm(self, a, w, c, n_out, k_in, stream_ptr, push=False, silu_mul=False, then=None):
        """`then` = (weights, n_out, k_in) of the GEMM that follows: its first weights are pulled into L2
        while this one drains (twm_gemm_args.next)."""
        nxt = None
        if then is not None:
            nxt = _lib.GemmArgs(M=self.rows, N=then[1], K=then[2], group_size=self.cfg.group_size, a_dtype=_lib.TWM_F16,
                                c_dtype=_lib.TWM_F32, packed=then[0][0].data_ptr(), scales=then[0][1].data_ptr(),
                                workspace=self.workspace.ptr, workspace_bytes=self.workspace.nbytes)
        args = _lib.GemmArgs(M=self.rows, N=n_out, K=k_in, group_size=self.cfg.group_size, a_dtype=_lib.TWM_F16,
                             c_dtype=_lib.TWM_F32 if c.dtype == torch.float32 else _lib.TWM_F16,
                             a=a.data_ptr(), lda=2 * k_in if silu_mul else k_in, packed=w[0].data_ptr(),
                             scales=w[1].data_ptr(), c=c.data_ptr(), ldc=n_out, workspace=self.workspace.ptr,
                             workspace_bytes=self.workspace.nbytes, flags=self.flags,
                             comm=self.comm.ptr if (push and self.comm is not None) else None,
                             a_prologue=_lib.TWM_A_SILU_MUL if silu_mul else _lib.TWM_A_PLAIN,
                             next=C.addressof(nxt) if nxt is not None else None)
        check(_lib.lib().twm_gemm_w4a16(C.byref(args), stream_ptr), "twm_gemm_w4a16")
        # kernels this call enqueued: the GEMM, and its activation pre-pass where the library uses one (from 9
        # rows always; from 3 rows with a push or on a matrix of 2^26 weights; from 2 rows with the prologue)
        m = self.rows
        staged = m >= 9 or (m >= 3 and ((push and self.comm is not None) or k_in * n_out >= 1 << 26)) or (silu_mul and m >= 2)
        self.launches += 2 if staged else 1

    def _join_and_norm(self, y_ptr, gamma_ptr, stream_ptr) -> None:
        """The summed output of the last row-parallel GEMM joins the residual stream, then RMSNorm."""
        lib, cfg = _lib.lib(), self.cfg
        if self.comm is not None:
            check(lib.twm_allreduce_add_rmsnorm(y_ptr, self.x.data_ptr(), self.comm.ptr, gamma_ptr, self.rows, cfg.hidden,
                                                cfg.eps, self.flags, stream_ptr), "twm_allreduce_add_rmsnorm")
        else:
            check(lib.twm_add_rmsnorm(y_ptr, self.x.data_ptr(), self.part.data_ptr(), gamma_ptr, self.rows, cfg.hidden,
                                      cfg.eps, self.flags, stream_ptr), "twm_add_rmsnorm")

    def attn_phase(self, li: int, stream_ptr: int) -> None:
        """Norm, column-parallel QKV, RoPE/append, attention, row-parallel o: leaves this rank's
        partial o output in `part` (to be summed over ranks) or, with `comm`, in every rank's slot."""
        lib, cfg, fl, m, lw, hd = _lib.lib(), self.cfg, self.flags, self.rows, self.layers[li], self.cfg.head_dim
        if li == 0:
            check(lib.twm_rmsnorm(self.normed.data_ptr(), self.x.data_ptr(), lw.attn_norm.data_ptr(), m, cfg.hidden,
                                  cfg.eps, fl, stream_ptr), "twm_rmsnorm")
        else:           # the previous layer's summed down output joins the residual stream here
            self._join_and_norm(self.normed.data_ptr(), lw.attn_norm.data_ptr(), stream_ptr)
        self._gemm(self.normed, lw.wqkv, self.qkv, self.spec.n_qkv, cfg.hidden, stream_ptr,            # column-parallel
                   then=(lw.wo, cfg.hidden, self.hq * hd))
        if li == 0:      # cos/sin of the step's position, once for all layers
            check(lib.twm_rope_table(self.rope_table.data_ptr(), self.pos.data_ptr(), hd, cfg.rope_theta, fl, stream_ptr),
                  "twm_rope_table")
            self.launches += 1
        check(lib.twm_attn_decode_rope(self.attn.data_ptr(), self.qkv.data_ptr(),
                                       lw.bqkv.data_ptr() if lw.bqkv is not None else None, self.rope_table.data_ptr(),
                                       self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(), m, self.hq, self.hk, hd,
                                       self.pos.data_ptr(), self.cache_len.data_ptr(), cfg.max_seq,
                                       self.attn_scratch.data_ptr(), self.attn_scratch.numel(), fl, stream_ptr),
              "twm_attn_decode_rope")
        self.launches += 3
        self._gemm(self.attn, lw.wo, self.part, cfg.hidden, self.hq * hd, stream_ptr, push=True,        # row-parallel
                   then=(lw.wgu, self.spec.n_gu, cfg.hidden))

    def ffn_phase(self, li: int, stream_ptr: int) -> None:
        """Add the all-reduced o output, norm, column-parallel gate+up, SwiGLU, row-parallel down:
        leaves this rank's partial down output in `part`."""
        lib, cfg, fl, m, lw = _lib.lib(), self.cfg, self.flags, self.rows, self.layers[li]
        self._join_and_norm(self.normed.data_ptr(), lw.ffn_norm.data_ptr(), stream_ptr)
        nl = self.layers[(li + 1) % len(self.layers)]
        after_down = (nl.wqkv, self.spec.n_qkv, cfg.hidden)
        self._gemm(self.normed, lw.wgu, self.gate_up, self.spec.n_gu, cfg.hidden, stream_ptr,            # column-parallel
                   then=(lw.w_down, cfg.hidden, self.spec.n_gu // 2))
        if m <= 32:     # the down GEMM's activation reader (one row) or its staging pre-pass (up to 32) takes
                        # silu(gate) * up on the fly: the same bits as the separate pass
            self.launches += 1
            self._gemm(self.gate_up, lw.w_down, self.part, cfg.hidden, self.spec.n_gu // 2, stream_ptr, push=True, silu_mul=True,
                       then=after_down)
            return
        check(lib.twm_silu_mul(self.act.data_ptr(), self.gate_up.data_ptr(), m, self.spec.n_gu // 2, fl, stream_ptr),
              "twm_silu_mul")
        self.launches += 2
        self._gemm(self.act, lw.w_down, self.part, cfg.hidden, self.spec.n_gu // 2, stream_ptr, push=True,   # row-parallel
                   then=after_down)

    def finish(self, stream_ptr: int) -> None:
        """The last layer's summed down output joins the residual stream."""
        self._join_and_norm(None, None, stream_ptr)
        self.launches += 1

    def forward(self, stream_ptr: int) -> None:
        """Enqueue the whole stack on the stream: x holds the input activations and, afterwards,
        the output.  Two all-reduces per layer, each on the [rows, hidden] FP32 partial."""
        self.launches = 0
        for li in range(len(self.layers)):
            self.attn_phase(li, stream_ptr)
            if self.comm is None:
                self.all_reduce(self.part)
            self.ffn_phase(li, stream_ptr)
            if self.comm is None:
                self.all_reduce(self.part)
        self.finish(stream_ptr)
