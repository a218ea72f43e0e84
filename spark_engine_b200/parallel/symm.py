"""Symmetric peer-memory arena and the collectives built on it.

One process per GPU.  Every rank allocates an arena of the same size with cudaMalloc, exports it with
cudaIpcGetMemHandle, the handles travel through torch.distributed (NCCL or gloo, plumbing only) and every
rank maps every peer's arena; kernels then address peers[p] + offset directly (NVLink P2P loads/stores).
Regions are carved out of the arena identically on all ranks, so one offset names the same buffer
everywhere.  Each collective owns a flag region and a monotonically increasing sequence number.

The reference has an RDMA transport with the same contract (fixed rank-order fp32 sums, bitwise identical
on all ranks, send-only + fused consumer: engine-rs/shim/rdma_arn.cu:84-125, tp.rs:299-356); its topology
code (links, GIDs, proxy threads) has no counterpart on an NVSwitch box.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import cuda as cu

vp, i32, i64, u32, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_uint, C.c_float


class CommCtx(C.Structure):
    _fields_ = [("peers", vp * 8), ("rank", i32), ("world", i32), ("wait_ns", C.c_ulonglong), ("status", vp)]


class ArRows(C.Structure):
    _fields_ = [("c", CommCtx), ("slot_off", i64), ("flag_off", i64), ("seq", u32), ("rows_cap", i32), ("R", i32),
                ("N", i32), ("inp", vp), ("in_f32", i32), ("counter", vp), ("res", vp), ("norm_w", vp), ("eps", f32),
                ("out", vp), ("out_f32", i32), ("seq_ptr", vp),
                ("moe_y", vp), ("moe_w", vp), ("moe_ids", vp), ("moe_slots", i32), ("moe_shared", vp), ("moe_sg", vp),
                ("ll_off", i64)]


class ArMoe(C.Structure):
    _fields_ = [("y", vp), ("w", vp), ("ids", vp), ("slots", i32), ("shared", vp), ("sg", vp)]


class HostPush(C.Structure):
    _fields_ = [("peers", vp * 8), ("slot_off", i64), ("flag_off", i64), ("rank", i32), ("world", i32),
                ("rows_per_rank", i32), ("seq", u32), ("counter", vp), ("seq_ptr", vp)]


class EpLayout(C.Structure):
    _fields_ = [("slab_off", i64), ("count_off", i64), ("flag_off", i64), ("ret_off", i64), ("ret_flag_off", i64),
                ("cap", i32), ("row_bytes", i32), ("seq_ptr", vp)]


_SIGS = {
    "spark_arena_alloc": ([i64], vp), "spark_arena_free": ([vp], None),
    "spark_ipc_get_handle": ([vp, vp], i32), "spark_ipc_open_handle": ([vp], vp), "spark_ipc_close": ([vp], None),
    "spark_comm_barrier": ([vp, i64, u32, vp], i32),
    "spark_allreduce_rows": ([vp, i64, i64, u32, i32, i32, i32, vp, i32, vp, vp, vp, f32, vp, i32, vp, vp, vp, i64], i32),
    "spark_allreduce_tail": ([vp, i64, i64, i32, i32, i32, vp, vp, vp, f32, vp, i32, vp, vp, i64], i32),
    "spark_tp_argmax": ([vp, i64, i64, vp, vp, i32, vp, i32, i32, i32, vp, vp, vp, vp], i32),
    "spark_rs_ag_rows": ([vp, i64, i64, i64, i64, u32, i32, i32, i32, vp, i32, vp, vp, vp, f32, i32, vp, vp], i32),
    "spark_ag_push": ([vp, vp, i32, i32, i64, i64, u32, vp, vp, vp], i32),
    "spark_seq_bump": ([vp, vp], i32),
    "spark_wait_flags": ([vp, i64, u32, vp], i32),
    "spark_wait_flags_dev": ([vp, i64, vp, i32, vp], i32),
    "spark_gemm_bf16_push_rs": ([vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, vp], i32),
    "spark_gemm_bf16_ag": ([vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, u32, i32, i32, i32, C.c_ulonglong, vp, vp, vp], i32),
    "spark_ep_row_bytes": ([i32], i32),
    "spark_ep_dispatch": ([vp, vp, u32, vp, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp], i32),
    "spark_ep_empty": ([vp, vp, u32, i32, vp], i32),
    "spark_ep_recv": ([vp, vp, u32, i32, vp, vp, vp, vp, i32, vp], i32),
    "spark_ep_combine_push": ([vp, vp, u32, i32, i32, vp, vp, vp, vp, i32, vp], i32),
    "spark_ep_combine_reduce": ([vp, vp, u32, i32, i32, i32, vp, vp, vp, vp], i32),
    "spark_exl3_gemv": None,
}
_bound = False


def _lib():
    global _bound
    lib = cu.lib()
    if not _bound:
        dll = lib._dll
        for name, sig in _SIGS.items():
            if sig is None:
                continue
            fn = getattr(dll, name)
            fn.argtypes, fn.restype = sig
        _bound = True
    return lib


class _DevPtrTensor:
    """Zero-copy torch view of raw device memory through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class Arena:
    """Arena of `nbytes` on every rank of `group`, with all peers mapped."""

    def __init__(self, nbytes: int, group=None, wait_ms: float = 1000.0):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        assert self.world <= 8
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        lib = _lib()
        self.base = lib._dll.spark_arena_alloc(self.nbytes)
        if not self.base:
            raise MemoryError("arena allocation failed")
        self.local = torch.as_tensor(_DevPtrTensor(self.base, self.nbytes), device=self.device)
        self.peer_ptrs = [0] * 8
        self.peer_ptrs[self.rank] = self.base
        self._opened = []
        if self.world > 1:
            handle = (C.c_ubyte * 64)()
            assert lib._dll.spark_ipc_get_handle(self.base, handle) == 0
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device)
            allh = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(allh, mine, group=group)
            for p in range(self.world):
                if p == self.rank:
                    continue
                buf = (C.c_ubyte * 64)(*allh[p].cpu().tolist())
                ptr = lib._dll.spark_ipc_open_handle(buf)
                if not ptr:
                    raise RuntimeError(f"cudaIpcOpenMemHandle failed for rank {p}")
                self.peer_ptrs[p] = ptr
                self._opened.append(ptr)
        self.ctx = CommCtx()
        for i in range(8):
            self.ctx.peers[i] = self.peer_ptrs[i]
        self.ctx.rank, self.ctx.world = self.rank, self.world
        self.ctx.wait_ns = int(wait_ms * 1e6)
        self.ctx.status = cu.status_word(self.device).data_ptr()
        self._top = 0
        self.regions: Dict[str, tuple] = {}
        self.seqs: Dict[str, int] = {}
        self._counters = torch.zeros(64, dtype=torch.int32, device=self.device)
        self._n_counters = 0
        self._seq_tensors = []
        self.flag_barrier = self.region("barrier_flags", 8 * 4)
        self.barrier()

    # -------------------------------------------------------------------------------------------
    def region(self, name: str, nbytes: int) -> int:
        """Offset of a named region (same on every rank: regions must be created in the same order)."""
        if name in self.regions:
            off, n = self.regions[name]
            assert n >= nbytes, f"region {name} too small"
            return off
        off = (self._top + 255) // 256 * 256
        assert off + nbytes <= self.nbytes, f"arena exhausted allocating {name} ({nbytes} bytes)"
        self._top = off + nbytes
        self.regions[name] = (off, nbytes)
        return off

    def view(self, off: int, nbytes: int, dtype=torch.uint8) -> torch.Tensor:
        return self.local[off: off + nbytes].view(dtype)

    def counter(self) -> int:
        """Pointer to a fresh zeroed device int (cross-CTA arrival counter)."""
        assert self._n_counters < 62
        p = self._counters[self._n_counters:].data_ptr()
        self._n_counters += 2
        return p

    def seq_counter(self) -> torch.Tensor:
        """Device-side sequence counter of one channel (kernels use value+1 and store it back, so a captured
        graph can be replayed)."""
        t = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._seq_tensors.append(t)
        return t

    def next_seq(self, name: str) -> int:
        self.seqs[name] = self.seqs.get(name, 0) + 1
        return self.seqs[name]

    def barrier(self):
        seq = self.next_seq("barrier")
        rc = _lib()._dll.spark_comm_barrier(C.byref(self.ctx), self.flag_barrier, seq, cu.stream())
        cu.check(rc, "spark_comm_barrier")

    def status(self) -> tuple:
        return cu.read_status(self.device)

    def close(self):
        torch.cuda.synchronize()
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)
        for p in self._opened:
            _lib()._dll.spark_ipc_close(p)
        self._opened = []
        if self.base:
            _lib()._dll.spark_arena_free(self.base)
            self.base = 0


class FusedAllReduce:
    """One-shot all-reduce of <= rows_cap rows of width N, optionally fused with residual add + RMSNorm,
    and usable as the epilogue of the EXL3 GEMV (`gemv_fused`)."""

    def __init__(self, arena: Arena, name: str, rows_cap: int, N: int):
        self.a, self.name, self.rows_cap, self.N = arena, name, rows_cap, N
        W = arena.world
        self.slot_off = arena.region(name + ".slots", 2 * W * rows_cap * N * 4)
        self.flag_off = arena.region(name + ".flags", 8 * 4)
        self.counter = arena.counter()
        self.seq = arena.seq_counter()
        # decode rounds (<= 16 rows): 8-byte {value, sequence} words, no flags (comm.cu `allreduce_rows_ll_kernel`)
        self.ll_off = -1
        if os.environ.get("SPARK_AR_LL", "1") == "1" and N <= 8192:
            nb = 2 * W * 16 * N * 8
            self.ll_off = arena.region(name + ".ll", nb)     # (the arena is zero-filled: below every live sequence number)

    def _args(self, R, inp, res, norm_w, eps, out) -> ArRows:
        ar = ArRows()
        ar.c = self.a.ctx
        ar.slot_off, ar.flag_off, ar.seq = self.slot_off, self.flag_off, 0
        ar.seq_ptr = self.seq.data_ptr()
        ar.rows_cap, ar.R, ar.N = self.rows_cap, R, self.N
        ar.inp = cu.P(inp)
        ar.in_f32 = int(inp is not None and inp.dtype == torch.float32)
        ar.counter = self.counter
        ar.res, ar.norm_w, ar.eps = cu.P(res), cu.P(norm_w), float(eps)
        ar.out, ar.out_f32 = cu.P(out), int(out.dtype == torch.float32)
        ar.ll_off = self.ll_off if R <= 16 else -1
        return ar

    def __call__(self, x, res: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                 eps: float = 1e-6, out_dtype=torch.bfloat16) -> torch.Tensor:
        """`x`: this rank's partial rows [R, N], or the uncombined expert outputs of a decode round (`cu.PendingMoe`):
        the slot-order combine then happens inside the push."""
        moe = None
        if isinstance(x, cu.PendingMoe):
            pm = x
            R, N = pm.R, pm.H
            moe = ArMoe()
            moe.y, moe.w, moe.ids, moe.slots = cu.P(pm.y), cu.P(pm.wts), cu.P(pm.ids), pm.slots
            moe.shared, moe.sg = cu.P(pm.shared), cu.P(pm.sg)
            dev, x = pm.y.device, None
        else:
            R, N = x.shape
            dev, x = x.device, x.contiguous()
        assert N == self.N and R <= self.rows_cap
        out = torch.empty(R, N, dtype=out_dtype, device=dev)
        ar = self._args(R, x, res, norm_w, eps, out)
        rc = _lib()._dll.spark_allreduce_rows(C.byref(ar.c), ar.slot_off, ar.flag_off, ar.seq, ar.rows_cap, R, N, ar.inp,
                                              ar.in_f32, ar.counter, ar.res, ar.norm_w, ar.eps, ar.out, ar.out_f32,
                                              cu.stream(), ar.seq_ptr, C.byref(moe) if moe is not None else None,
                                              C.c_longlong(ar.ll_off))
        cu.check(rc, "spark_allreduce_rows")
        return out

    def gemv_fused(self, x: torch.Tensor, w, res=None, norm_w=None, eps=1e-6, act=0, limit=0.0,
                   out_dtype=torch.bfloat16) -> torch.Tensor:
        """y = allreduce(x @ W_shard^T) (+ res)(-> RMSNorm): the row-parallel EXL3 GEMV pushes its strips straight into
        every rank's slots from its epilogue (no local round trip of the partial rows) and raises the flag; a tail
        launch with one CTA per row reduces."""
        from ..quant.formats import Exl3Weight
        assert isinstance(w, Exl3Weight) and not w.experts and w.n == self.N
        R = x.shape[0]
        out = torch.empty(R, self.N, dtype=out_dtype, device=x.device)
        ar = self._args(R, None, res, norm_w, eps, out)
        S = cu._pick_slices(w.k)
        rc = cu.lib().spark_exl3_gemv(cu.P(x), x.stride(0), cu.P(w.trellis), cu.P(w.suh), cu.P(w.svh), 0, 0, 0, None,
                                      self.N, 0, None, None, 1, R, w.k, w.n, S, act, float(limit),
                                      0 if w.kind == "mul1" else 1, cu.stream(), C.addressof(ar), 0)
        cu.check(rc, "spark_exl3_gemv(fused all-reduce)")
        rc = _lib()._dll.spark_allreduce_tail(C.byref(ar.c), ar.slot_off, ar.flag_off, ar.rows_cap, R, self.N, ar.counter, ar.res,
                                              ar.norm_w, ar.eps, ar.out, ar.out_f32, cu.stream(), ar.seq_ptr,
                                              C.c_longlong(ar.ll_off))
        cu.check(rc, "spark_allreduce_tail")
        self._keep = ar
        return out


class PacketArgmax:
    """Vocabulary-parallel greedy sampling: local two-stage arg-max, (value, global id) packets pushed to every rank,
    winner picked in rank order (ties -> lowest id); two launches, no host work, replayable under CUDA graphs."""

    def __init__(self, arena: Arena, name: str, rows_cap: int = 64):
        self.a, self.rows_cap = arena, rows_cap
        self.slot_off = arena.region(name + ".packets", 2 * arena.world * rows_cap * 8)
        self.flag_off = arena.region(name + ".flags", 8 * 4)
        self.counter = arena.counter()
        self.seq = arena.seq_counter()

    def __call__(self, logits: torch.Tensor, vocab_off: int) -> torch.Tensor:
        R, V = logits.shape
        assert R <= self.rows_cap and logits.dtype == torch.float32
        logits = logits.contiguous()
        ids = torch.empty(R, dtype=torch.int32, device=logits.device)
        pv = cu.scratch("tp_argmax_v", R * 64, torch.float32, logits.device)
        pi = cu.scratch("tp_argmax_i", R * 64, torch.int32, logits.device)
        rc = _lib()._dll.spark_tp_argmax(C.byref(self.a.ctx), self.slot_off, self.flag_off, self.seq.data_ptr(), self.counter,
                                         self.rows_cap, cu.P(logits), R, V, vocab_off, cu.P(pv), cu.P(pi), cu.P(ids), cu.stream())
        cu.check(rc, "spark_tp_argmax")
        return ids


class RowParallelGemm:
    """Prefill: row-parallel tcgen05 GEMM whose epilogue pushes fp32 partial tiles to the owner rank of each row
    block (reduce-scatter), owners sum in rank order (+ residual + RMSNorm) and all-gather the bf16 rows."""

    def __init__(self, arena: Arena, name: str, rows_cap: int, N: int):
        W = arena.world
        self.a, self.name, self.N = arena, name, N
        self.rpr_cap = (rows_cap + W - 1) // W
        self.slot_off = arena.region(name + ".slots", W * self.rpr_cap * N * 4)
        self.out_off = arena.region(name + ".out", W * self.rpr_cap * N * 2)
        self.flag_rs = arena.region(name + ".frs", 32)
        self.flag_ag = arena.region(name + ".fag", 32)
        self.counters = torch.zeros(4, dtype=torch.int32, device=arena.device)
        self.seq = arena.seq_counter()

    def __call__(self, x, w, res_owned=None, norm_w=None, eps=1e-6, fused=True) -> torch.Tensor:
        """x [M, K_shard] bf16, w [N, K_shard] bf16 -> gathered result rows [M, N] bf16 (view into the arena)."""
        a = self.a
        W = a.world
        M, K = x.shape
        rpr = (M + W - 1) // W
        assert rpr <= self.rpr_cap
        Mp = rpr * W
        seq = 0
        lib = _lib()._dll
        if fused:
            hp = HostPush()
            for i in range(8):
                hp.peers[i] = a.peer_ptrs[i]
            hp.slot_off, hp.flag_off, hp.rank, hp.world = self.slot_off, self.flag_rs, a.rank, W
            hp.rows_per_rank, hp.seq, hp.counter = rpr, seq, self.counters.data_ptr()
            hp.seq_ptr = self.seq.data_ptr()
            rc = lib.spark_gemm_bf16_push_rs(cu.P(x), cu.P(w), Mp if Mp == M else M, self.N, K, x.stride(0), w.stride(0), 1,
                                             C.byref(hp), cu.P(cu.status_word(x.device)), cu.stream())
            cu.check(rc, "spark_gemm_bf16_push_rs")
            push_only = 2
            inp = None
        else:
            return self.rows(cu.gemm_bf16(x, w, out_f32=True), res_owned, norm_w, eps)
        rc = lib.spark_rs_ag_rows(C.byref(a.ctx), self.slot_off, self.out_off, self.flag_rs, self.flag_ag, seq, Mp,
                                  self.N, rpr, cu.P(inp), 1, self.counters[1:].data_ptr(), cu.P(res_owned), cu.P(norm_w),
                                  float(eps), push_only, cu.stream(), self.seq.data_ptr())
        cu.check(rc, "spark_rs_ag_rows")
        return a.view(self.out_off, Mp * self.N * 2, torch.bfloat16).view(Mp, self.N)[:M]

    def rows(self, part: torch.Tensor, res_owned=None, norm_w=None, eps=1e-6) -> torch.Tensor:
        """Reduce-scatter + (residual + RMSNorm on the owned row block) + all-gather of precomputed partial rows
        `part` [M, N] (fp32 or bf16): every rank ends with all M result rows in bf16 (a view into the arena, valid
        until the next call) and `res_owned` (this rank's block of the residual stream) updated in place."""
        a = self.a
        W = a.world
        M = part.shape[0]
        rpr = (M + W - 1) // W
        assert rpr <= self.rpr_cap and part.shape[1] == self.N
        Mp = rpr * W
        part = part.contiguous()
        if Mp != M:
            part = torch.cat((part, part.new_zeros(Mp - M, self.N)))
        rc = _lib()._dll.spark_rs_ag_rows(C.byref(a.ctx), self.slot_off, self.out_off, self.flag_rs, self.flag_ag, 0, Mp,
                                          self.N, rpr, cu.P(part), int(part.dtype == torch.float32),
                                          self.counters[1:].data_ptr(), cu.P(res_owned), cu.P(norm_w), float(eps), 0,
                                          cu.stream(), self.seq.data_ptr())
        cu.check(rc, "spark_rs_ag_rows")
        return a.view(self.out_off, Mp * self.N * 2, torch.bfloat16).view(Mp, self.N)[:M]


class AllGatherGemm:
    """Column-parallel GEMM with the all-gather of its row-sharded input fused in."""

    def __init__(self, arena: Arena, name: str, rows_cap: int, K: int):
        W = arena.world
        self.a, self.name, self.K = arena, name, K
        self.rpr_cap = (rows_cap + W - 1) // W
        self.buf_off = arena.region(name + ".gather", W * self.rpr_cap * K * 2)
        self.flag_off = arena.region(name + ".flags", 32)
        self.counter = arena.counter()
        self.seq = arena.seq_counter()

    def __call__(self, x_local, w, out_f32=False) -> torch.Tensor:
        """x_local [rows, K] bf16 (this rank's row block) ; w [N_shard, K] -> [world*rows, N_shard]."""
        a = self.a
        W = a.world
        rows, K = x_local.shape
        assert K == self.K and rows <= self.rpr_cap
        seq = 0
        lib = _lib()._dll
        rc = lib.spark_ag_push(C.byref(a.ctx), cu.P(x_local.contiguous()), rows, K, self.buf_off, self.flag_off, seq,
                               self.counter, cu.stream(), self.seq.data_ptr())
        cu.check(rc, "spark_ag_push")
        M, N = W * rows, w.shape[0]
        out = torch.empty(M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x_local.device)
        rc = lib.spark_gemm_bf16_ag(a.base + self.buf_off, cu.P(w), cu.P(out), M, N, K, w.stride(0), N, int(out_f32),
                                    a.base + self.flag_off, seq, rows, a.rank, W, a.ctx.wait_ns,
                                    cu.P(cu.status_word(x_local.device)), cu.stream(), self.seq.data_ptr())
        cu.check(rc, "spark_gemm_bf16_ag")
        cu.check(lib.spark_seq_bump(self.seq.data_ptr(), cu.stream()), "spark_seq_bump")
        return out


class ExpertParallel:
    """EP all-to-all: dispatch (router top-k + FP8 1x128 quant + scatter) and combine (gather + slot-order
    weighted sum)."""

    def __init__(self, arena: Arena, name: str, tokens_cap: int, H: int, E: int, top_k: int, cap_factor: float = 2.0):
        W = arena.world
        self.a, self.name, self.H, self.E, self.k, self.T_cap = arena, name, H, E, top_k, tokens_cap
        lib = _lib()._dll
        self.row_bytes = lib.spark_ep_row_bytes(H)
        self.cap = max(16, int(tokens_cap * top_k / W * cap_factor) + 16)
        self.cap = min(self.cap, tokens_cap * top_k)
        L = EpLayout()
        L.slab_off = arena.region(name + ".slab", W * self.cap * self.row_bytes)
        L.count_off = arena.region(name + ".count", 32)
        L.flag_off = arena.region(name + ".flag", 32)
        L.ret_off = arena.region(name + ".ret", tokens_cap * top_k * H * 2)
        L.ret_flag_off = arena.region(name + ".rflag", 32)
        L.cap, L.row_bytes = self.cap, self.row_bytes
        self.seq_dev = arena.seq_counter()
        L.seq_ptr = self.seq_dev.data_ptr()
        self.L = L
        dev = arena.device
        self.send_count = torch.zeros(8, dtype=torch.int32, device=dev)
        self.counters = torch.zeros(4, dtype=torch.int32, device=dev)
        self.max_rows = W * self.cap
        self.a_rows = torch.empty(self.max_rows, H, dtype=torch.bfloat16, device=dev)
        self.expert_local = torch.empty(self.max_rows, dtype=torch.int32, device=dev)
        self.meta = torch.empty(self.max_rows, 4, dtype=torch.int32, device=dev)
        self.total = torch.zeros(1, dtype=torch.int32, device=dev)

    def dispatch(self, x: torch.Tensor, logits: torch.Tensor):
        """x [T,H] bf16, logits [T,E] fp32 -> (wts [T,k], ids [T,k]); received rows land in self.a_rows[:total]."""
        a, lib = self.a, _lib()._dll
        T = x.shape[0]
        self.seq = 0
        wts = torch.empty(T, self.k, dtype=torch.float32, device=x.device)
        ids = torch.empty(T, self.k, dtype=torch.int32, device=x.device)
        if T == 0:
            rc = lib.spark_ep_empty(C.byref(a.ctx), C.byref(self.L), self.seq, 0, cu.stream())
        else:
            rc = lib.spark_ep_dispatch(C.byref(a.ctx), C.byref(self.L), self.seq, cu.P(x.contiguous()), T, self.H,
                                       cu.P(logits), logits.stride(0), self.E, self.k, cu.P(wts), cu.P(ids),
                                       cu.P(self.send_count), cu.P(self.counters), cu.stream())
        cu.check(rc, "spark_ep_dispatch")
        rc = lib.spark_ep_recv(C.byref(a.ctx), C.byref(self.L), self.seq, self.H, cu.P(self.a_rows), cu.P(self.expert_local),
                               cu.P(self.meta), cu.P(self.total), self.max_rows, cu.stream())
        cu.check(rc, "spark_ep_recv")
        return wts, ids

    def combine(self, y: torch.Tensor, wts: torch.Tensor, T: int, res: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y [>= total, H] bf16 expert outputs in received-row order -> out [T,H] bf16 (and res += out)."""
        a, lib = self.a, _lib()._dll
        rc = lib.spark_ep_combine_push(C.byref(a.ctx), C.byref(self.L), self.seq, self.H, self.k, cu.P(y), cu.P(self.meta),
                                       cu.P(self.total), self.counters[2:].data_ptr(), self.max_rows, cu.stream())
        cu.check(rc, "spark_ep_combine_push")
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=y.device)
        if T == 0:
            rc = lib.spark_wait_flags_dev(C.byref(a.ctx), self.L.ret_flag_off, self.seq_dev.data_ptr(), 0, cu.stream())
        else:
            rc = lib.spark_ep_combine_reduce(C.byref(a.ctx), C.byref(self.L), self.seq, T, self.H, self.k, cu.P(wts),
                                             cu.P(res), cu.P(out), cu.stream())
        cu.check(rc, "spark_ep_combine_reduce")
        cu.check(lib.spark_seq_bump(self.seq_dev.data_ptr(), cu.stream()), "spark_seq_bump")
        return out
