"""Fused Llama training engine for B200: the network as an explicit kernel schedule.

Instead of tracing modules through autograd and a compiler (the reference wraps its
``Transformer`` in FSDP2 + ``torch.compile``, src/zeroband/train.py:150-168, 208-211), the
engine owns flat parameter / gradient / optimizer buffers (see :mod:`.layout`) and runs forward,
backward and the optimizer as a fixed sequence of hand-written sm_100a kernels on one CUDA
stream, with the ZeRO-3 collectives on a second stream:

  forward   embedding -> L x [rmsnorm, fused QKV GEMM, RoPE, flash attention, wo GEMM (+residual
            epilogue), rmsnorm, fused w1|w3 GEMM, SwiGLU, w2 GEMM (+residual epilogue)]
  head      final rmsnorm, then per token chunk: logits GEMM, cross-entropy with in-place
            gradient, dgrad + wgrad GEMMs (logits never exist for more than one chunk)
  backward  per block: 4 dgrad + 4 wgrad GEMMs, SwiGLU bwd, flash attention bwd with the inverse
            RoPE folded into its last pass, 2 rmsnorm bwd (residual gradient folded in)
  update    per parameter group: reduce-scatter-by-pull + cast/scale + sum-of-squares, then one
            scalar all-reduce for the global norm, then sharded AdamW that pushes the new bf16
            values into every rank's replica (all-gather by push)

By default the bf16 parameter replica stays resident on every GPU (180 GB HBM makes ZeRO-3's re-gather
before every use unnecessary); what is sharded is everything fp32: master weights, AdamW moments
and the reduced gradient.

``reshard=True`` (the reference's ``train.reshard_after_forward``, src/zeroband/train.py:150-168) drops the
replica: every rank keeps only its bf16 row shards (symmetric memory) and a transformer block's weights
exist in full only while the block runs, in one of two block-sized buffers. In the forward the fused QKV
projection gathers its own operand (wq | wk | wv) inside the GEMM (csrc/gemm2_sm100.cu, all-gather fused
into the first consuming GEMM) while the rest of the NEXT block is fetched on the comm stream; in the
backward each block is re-gathered one block ahead. Embedding, final norm and head are gathered once per
optimizer step.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from .. import native
from ..models.llama import ModelArgs
from ..native import check, ptr, stream_ptr
from ..ops import attention as A
from ..ops import kernels as K
from .layout import ParamLayout, llama_layout

native.register_cuda_sigs({
    "pb_zero_max_segs": [],
    "pb_zero_cta_ranges": [native.i32, native.vp, native.i32, native.vp],
    "pb_zero_max_ranks": [],
    "pb_peer_barrier": [native.vp, native.i32, native.i32, native.i32, native.i32, native.vp, native.vp],
    "pb_allreduce_scalars": [native.vp, native.vp, native.i32, native.i32, native.i32, native.i32, native.vp, native.vp,
                             native.i32, native.vp, native.vp],
    "pb_zero_reduce_grads": [native.vp, native.i32, native.i32, native.i32, native.i32, native.vp, native.vp, native.vp,
                             native.vp, native.f32, native.vp, native.vp, native.i32, native.i32, native.vp],
    "pb_zero_adamw_gather": [native.vp, native.i32, native.i32, native.i32, native.vp, native.vp, native.vp, native.vp,
                             native.vp, native.vp, native.vp, native.f32, native.f32, native.f32, native.f32, native.f32,
                             native.i32, native.vp, native.f32, native.i32, native.vp],
    "pb_zero_push_params": [native.vp, native.i32, native.i32, native.i32, native.vp, native.vp, native.vp, native.vp,
                            native.i32, native.vp],
    "pb_zero_gather_segments": [native.vp, native.i32, native.i32, native.i32, native.vp, native.vp, native.vp, native.vp, native.vp,
                                native.i32, native.vp],
    "pb_gemm_bf16_allgather_parts": [native.vp, native.vp, native.vp, native.vp, native.vp, native.i32, native.i32, native.i32, native.i64,
                                     native.i64, native.i64, native.i64, native.i32, native.i32, native.i32, native.i32, native.i32,
                                     native.vp, native.vp, native.vp, native.vp, native.i32, native.i32, native.vp, native.vp],
})


class _SegArrays:
    """ctypes arrays describing the segments of one group (or of all groups) for one rank. Neighbouring
    segments that are contiguous both in the full buffer and in the shard buffer are merged (with one rank
    the whole model is a single segment)."""

    def __init__(self, segs):
        runs: list[list[int]] = []
        for s in segs:
            if s.numel <= 0:
                continue
            if runs and runs[-1][0] + runs[-1][2] == s.full_offset and runs[-1][1] + runs[-1][2] == s.shard_offset:
                runs[-1][2] += s.numel
            else:
                runs.append([s.full_offset, s.shard_offset, s.numel])
        self.n = len(runs)
        arr = C.c_longlong * max(self.n, 1)
        self.full = arr(*[r[0] for r in runs])
        self.shard = arr(*[r[1] for r in runs])
        self.numel = arr(*[r[2] for r in runs])
        self.total = sum(r[2] for r in runs)


class LocalComm:
    """Single-rank stand-in for the symmetric-memory communicator: buffers are ordinary tensors."""
    world = 1
    rank = 0

    def alloc(self, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
        return torch.zeros(numel, dtype=dtype, device=device)

    def peer_ptrs(self, t: torch.Tensor):
        return (C.c_void_p * 1)(t.data_ptr())

    def barrier(self, slot: int = 0, stream=None):
        pass

    def host_barrier(self):
        pass

    def allreduce_scalars(self, src: torch.Tensor, dst: torch.Tensor, n: int):
        dst[:n].copy_(src[:n])


class FusedLlama:
    """See module docstring. One instance per process / GPU."""

    def __init__(self, args: ModelArgs, device: torch.device | str = "cuda", comm=None, grad_dtype=torch.bfloat16,
                 ac_ckpt: bool | int = False, ce_chunk_tokens: int = 32768, z_mode: int = K.Z_NONE, z_weight: float = 0.0,
                 comm_ctas: int = 37, reshard: bool = False):
        self.args = args
        self.device = torch.device(device)
        self.comm = comm if comm is not None else LocalComm()
        self.world, self.rank = self.comm.world, self.comm.rank
        self.layout: ParamLayout = llama_layout(args, self.world)
        self.grad_dtype = grad_dtype
        self.ac_every = (1 if ac_ckpt is True else int(ac_ckpt)) if ac_ckpt else 0
        self.ce_chunk = ce_chunk_tokens
        self.z_mode, self.z_weight = z_mode, z_weight
        self.comm_ctas = comm_ctas
        lay = self.layout
        dev = self.device
        # re-gather mode needs peers to gather from; with one rank the "shard" is the whole model
        self.reshard = bool(reshard) and self.world > 1 and self.device.type == "cuda"
        # flat buffers --------------------------------------------------------------------------
        if not self.reshard:
            self.params = self.comm.alloc(lay.full_numel, torch.bfloat16, dev)   # replica, symmetric
        else:
            self.params = None
            self.param_shard = self.comm.alloc(lay.max_shard_numel, torch.bfloat16, dev)    # this rank's bf16 rows, symmetric
        self.grads = self.comm.alloc(lay.full_numel, grad_dtype, dev)             # local grads, symmetric
        n_shard = lay.shard_numel[self.rank]
        self.master = torch.zeros(n_shard, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(n_shard, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n_shard, dtype=torch.float32, device=dev)
        self.grad_shard = torch.zeros(n_shard, dtype=torch.float32, device=dev)
        self._peer_params = self.comm.peer_ptrs(self.params) if not self.reshard else None
        self._peer_grads = self.comm.peer_ptrs(self.grads)
        self._segs = [_SegArrays(lay.group_segments(self.rank, g)) for g in range(len(lay.groups))]
        max_segs = native.cuda().pb_zero_max_segs() if dev.type == "cuda" else 16
        assert all(s.n <= max_segs for s in self._segs)
        # all groups in one table: the reduce and the AdamW + push run as one launch each when it fits
        allsegs = _SegArrays([s for g in range(len(lay.groups)) for s in lay.group_segments(self.rank, g)])
        self._segs_step = [allsegs] if allsegs.n <= max_segs else self._segs
        self._partials = torch.zeros(4096, dtype=torch.float32, device=dev)
        self._norm_parts = torch.zeros(len(lay.groups), dtype=torch.float32, device=dev)   # sum of squares per group
        self._reduced_groups: set[int] = set()      # groups whose reduce-scatter is already in flight on the comm stream
        self.overlap_reduce = True                  # False: every group is reduced after the backward, on the main stream
        self._reduce_in_backward = False
        self._shard_opt = None         # set_shard_optimizer(): a torch optimizer on the shards instead of the AdamW kernel
        self._norm_local = torch.zeros(8, dtype=torch.float32, device=dev)
        self._norm_global = torch.zeros(8, dtype=torch.float32, device=dev)
        self.opt_step = 0
        self._accum = False            # gradients hold a partial sum from earlier micro-batches
        self._ws: dict[str, torch.Tensor] = {}
        self._rope = K.rope_table(args.max_seq_len * 2, args.head_dim, args.rope_theta, dev)
        self._seq_start_cache: dict[tuple[int, int], torch.Tensor] = {}
        self.comm_stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        # Weight-gradient GEMMs do not feed the input-gradient chain, so they can run on a stream of their own
        # (PRIME_B200_WGRAD_STREAM=1): the SMs a persistent GEMM leaves idle in its last wave are then open to CTAs of the
        # other stream's kernel. Hazards are handled per buffer: a wgrad records an event for the tensors it reads, and the
        # main stream waits for that event before the next kernel that overwrites one of them. Off by default: measured on
        # the 150M step it changes nothing (109.2-109.4 ms with, 109.1-109.3 ms without) because the step runs against the
        # 1000 W power cap (SM clock 1.48-1.54 GHz of 1.965), not against idle SMs.
        import os
        self.wgrad_stream = torch.cuda.Stream(device=dev) if (dev.type == "cuda" and os.environ.get("PRIME_B200_WGRAD_STREAM", "0") == "1") \
            else None
        self._readers: dict[int, torch.cuda.Event] = {}
        # parameter views -----------------------------------------------------------------------
        self.w: dict[str, torch.Tensor] = {}
        self.g: dict[str, torch.Tensor] = {}
        for p in lay.params:
            if not self.reshard:
                self.w[p.name] = self.params[p.offset: p.offset + p.numel].view(p.shape)
            self.g[p.name] = self.grads[p.offset: p.offset + p.numel].view(p.shape)
        D, F, hd, H, KV = args.dim, args.hidden_dim, args.head_dim, args.n_heads, args.kv_heads
        self.wqkv, self.gqkv, self.w13, self.g13 = [], [], [], []
        for i in range(args.n_layers):
            q = lay.params[lay.by_name[f"layers.{i}.attention.wq.weight"]]
            n = (H + 2 * KV) * hd * D
            self.wqkv.append(self.params[q.offset: q.offset + n].view((H + 2 * KV) * hd, D) if not self.reshard else None)
            self.gqkv.append(self.grads[q.offset: q.offset + n].view((H + 2 * KV) * hd, D))
            w1 = lay.params[lay.by_name[f"layers.{i}.feed_forward.w1.weight"]]
            self.w13.append(self.params[w1.offset: w1.offset + 2 * F * D].view(2 * F, D) if not self.reshard else None)
            self.g13.append(self.grads[w1.offset: w1.offset + 2 * F * D].view(2 * F, D))
        if self.reshard:
            self._init_reshard()

    # ------------------------------------------------------------------------------------------
    # re-gather mode: block-sized gathered buffers instead of a resident replica
    # ------------------------------------------------------------------------------------------
    def _init_reshard(self) -> None:
        lay, a, dev = self.layout, self.args, self.device
        L = a.n_layers
        self._peer_shards = self.comm.peer_ptrs(self.param_shard)
        blk = max(lay.groups[1 + i].full_end - lay.groups[1 + i].full_start for i in range(L))
        self._gbuf = [torch.empty(blk, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self._gbuf_holds = [-1, -1]                 # block whose weights a buffer holds (complete or in flight)
        self._gbuf_whole = [False, False]           # ... including the other ranks' wq | wk | wv rows
        self._gbuf_ready: list[torch.cuda.Event | None] = [None, None]    # comm-stream event: the buffer's gather is done
        self._gbuf_free: list[torch.cuda.Event | None] = [None, None]     # main-stream event: the block that used it is done
        g0, gh = lay.groups[0], lay.groups[L + 1]
        self._root_off = {0: 0, L + 1: (g0.full_end - g0.full_start + 63) // 64 * 64}
        self._root_buf = torch.empty(self._root_off[L + 1] + gh.full_end - gh.full_start, dtype=torch.bfloat16, device=dev)
        self._root_fresh = False                    # embedding / final norm / head hold the current parameters
        for g in (0, L + 1):
            for pi in lay.groups[g].params:
                p = lay.params[pi]
                o = self._root_off[g] + p.offset - lay.groups[g].full_start
                self.w[p.name] = self._root_buf[o: o + p.numel].view(p.shape)
        # copy tables: (owner rank, offset in its shard buffer) -> offset in the gathered buffer
        H, KV, hd = a.n_heads, a.kv_heads, a.head_dim
        self._tab_all, self._tab_rest, self._k2 = {}, {}, {}
        for g in range(len(lay.groups)):
            rows_all, rows_rest = [], []
            fused = set()
            if 1 <= g <= L:
                names = [f"layers.{g - 1}.attention.{n}.weight" for n in ("wq", "wk", "wv")]
                parts = [lay.params[lay.by_name[n]] for n in names]
                rpr = [-(-p.rows // self.world) for p in parts]
                n_tot = sum(p.rows for p in parts)
                ok = all(p.rows % self.world == 0 and r % 32 == 0 for p, r in zip(parts, rpr)) and n_tot % 256 == 0 and a.dim % 8 == 0
                if ok:
                    fused = {lay.by_name[n] for n in names}
                    segs = [lay.segments[self.rank][lay.by_name[n]] for n in names]
                    self._k2[g] = {
                        "rows": (C.c_int * 3)(*[p.rows for p in parts]), "rpr": (C.c_int * 3)(*rpr),
                        "off": (C.c_longlong * 3)(*[s_.shard_offset - segs[0].shard_offset for s_ in segs]),
                        "shards": (C.c_void_p * self.world)(*[pp + segs[0].shard_offset * 2 for pp in self._peer_shards]),
                        "n": n_tot, "dst_off": parts[0].offset - lay.groups[g].full_start,
                        "counters": torch.zeros(n_tot // 256, dtype=torch.int32, device=dev), "calls": 0}
            base = lay.groups[g].full_start
            for pi in lay.groups[g].params:
                for r in range(self.world):
                    sgm = lay.segments[r][pi]
                    if sgm.numel <= 0:
                        continue
                    row = (r, sgm.shard_offset, sgm.full_offset - base, sgm.numel)
                    rows_all.append(row)
                    if pi not in fused or r == self.rank:      # the fused QKV GEMM fetches the other ranks' rows itself
                        rows_rest.append(row)
            self._tab_all[g] = self._mk_tables(rows_all)
            self._tab_rest[g] = self._mk_tables(rows_rest)

    @staticmethod
    def _mk_tables(rows, limit: int = 128):
        out = []
        for i in range(0, len(rows), limit):
            ch = rows[i: i + limit]
            n = len(ch)
            out.append((n, (C.c_int * n)(*[r[0] for r in ch]), (C.c_longlong * n)(*[r[1] for r in ch]),
                        (C.c_longlong * n)(*[r[2] for r in ch]), (C.c_longlong * n)(*[r[3] for r in ch])))
        return out

    def _gather_into(self, tables, dst: torch.Tensor, stream) -> None:
        lib = native.cuda()
        for n, owner, src, dsto, numel in tables:
            check(lib.pb_zero_gather_segments(self._peer_shards, self.world, self.rank, n, owner, src, dsto, numel, ptr(dst),
                                              self.comm_ctas * 2, stream_ptr(stream)), "pb_zero_gather_segments")

    def _bind_block(self, i: int, buf: torch.Tensor) -> None:
        """Point the weight views of block ``i`` at the gathered buffer that holds it."""
        lay, a = self.layout, self.args
        base = lay.groups[1 + i].full_start
        for pi in lay.groups[1 + i].params:
            p = lay.params[pi]
            self.w[p.name] = buf[p.offset - base: p.offset - base + p.numel].view(p.shape)
        D, F, hd, H, KV = a.dim, a.hidden_dim, a.head_dim, a.n_heads, a.kv_heads
        q = lay.params[lay.by_name[f"layers.{i}.attention.wq.weight"]]
        self.wqkv[i] = buf[q.offset - base: q.offset - base + (H + 2 * KV) * hd * D].view((H + 2 * KV) * hd, D)
        w1 = lay.params[lay.by_name[f"layers.{i}.feed_forward.w1.weight"]]
        self.w13[i] = buf[w1.offset - base: w1.offset - base + 2 * F * D].view(2 * F, D)

    def _fetch_block(self, i: int, whole: bool) -> None:
        """Start the gather of block ``i`` on the comm stream into the buffer of its parity (a no-op when the buffer still
        holds the block). ``whole`` = every weight (backward); otherwise everything except the other ranks' wq | wk | wv
        rows, which the fused QKV projection fetches inside its GEMM."""
        slot = i % 2
        if self._gbuf_holds[slot] == i and (not whole or self._gbuf_whole[slot]):
            return
        cs = self.comm_stream
        if self._gbuf_free[slot] is not None:
            cs.wait_event(self._gbuf_free[slot])        # the block that last used this buffer has finished on the main stream
        tables = self._tab_all[1 + i] if (whole or (1 + i) not in self._k2) else self._tab_rest[1 + i]
        self._gather_into(tables, self._gbuf[slot], cs)
        ev = torch.cuda.Event()
        ev.record(cs)
        self._gbuf_ready[slot] = ev
        self._gbuf_holds[slot] = i
        self._gbuf_whole[slot] = whole or (1 + i) not in self._k2

    def _use_block(self, i: int) -> None:
        """Main stream: block ``i``'s gathered weights are about to be read."""
        slot = i % 2
        assert self._gbuf_holds[slot] == i
        torch.cuda.current_stream().wait_event(self._gbuf_ready[slot])
        self._bind_block(i, self._gbuf[slot])

    def _release_block(self, i: int) -> None:
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self._gbuf_free[i % 2] = ev

    def _ensure_root(self) -> None:
        if self._root_fresh:
            return
        L = self.args.n_layers
        main = torch.cuda.current_stream()
        for g in (0, L + 1):
            self._gather_into(self._tab_all[g], self._root_buf[self._root_off[g]:], main)
        self._root_fresh = True

    # ------------------------------------------------------------------------------------------
    # parameter I/O
    # ------------------------------------------------------------------------------------------
    def shard_view(self, buf: torch.Tensor, name: str) -> torch.Tensor:
        """This rank's dim-0 slice of parameter ``name`` inside a shard-layout buffer."""
        lay = self.layout
        i = lay.by_name[name]
        s = lay.segments[self.rank][i]
        p = lay.params[i]
        return buf[s.shard_offset: s.shard_offset + s.numel].view((s.row_end - s.row_start,) + p.shape[1:])

    def named_master_shards(self):
        for p in self.layout.params:
            yield p.name, self.shard_view(self.master, p.name)

    def set_shard_optimizer(self, factory) -> torch.optim.Optimizer:
        """Replace the sharded AdamW kernel by a ``torch.optim.Optimizer`` that works on this rank's shards: ``factory``
        gets one ``nn.Parameter`` per model parameter whose data is the rank's dim-0 slice of the fp32 master weights
        (a view, so the update lands in place) and whose ``.grad`` is the matching view of the reduced, averaged fp32
        gradient shard. The engine still does forward / backward, the reduce-scatter, the global-norm clip and the bf16
        all-gather; the optimizer sees exactly what FSDP2 would hand a sharded optimizer (each rank's rows of every
        parameter), which is how a fully-sharded Shampoo / SOAP preconditions: per rank, on its own block of rows."""
        params = []
        for name, shard in self.named_master_shards():
            q = torch.nn.Parameter(shard, requires_grad=True)
            q.grad = self.shard_view(self.grad_shard, name)
            params.append(q)
        self._shard_params = params
        self._shard_opt = factory([q for q in params if q.numel() > 0])
        return self._shard_opt

    def _shard_optimizer_update(self, lr: float, max_norm: float) -> None:
        """grad_shard holds this rank's averaged fp32 gradients and _norm_global[0] the squared global norm."""
        if max_norm > 0:
            coef = (max_norm / (self._norm_global[0].sqrt() + 1e-6)).clamp(max=1.0)
            self.grad_shard.mul_(coef)
        for group in self._shard_opt.param_groups:
            group["lr"] = lr
        self._shard_opt.step()
        self.publish_params()          # bf16 copies of the new master rows into every rank's replica

    @torch.no_grad()
    def load_from_module(self, model: torch.nn.Module) -> None:
        """Copy fp32 weights of an eager ``Transformer`` into the master shard, then publish bf16."""
        sd = dict(model.named_parameters())
        for p in self.layout.params:
            s = self.layout.segments[self.rank][self.layout.by_name[p.name]]
            src = sd[p.name].detach()[s.row_start: s.row_end]
            self.shard_view(self.master, p.name).copy_(src.to(self.device, torch.float32))
        self.publish_params()

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float | None = None) -> None:
        """Plain N(0, std) initialisation (norm weights = 1) generated shard-by-shard on device;
        every rank draws only the rows it owns from a per-parameter seeded generator."""
        std = self.args.init_std if std is None else std
        for idx, p in enumerate(self.layout.params):
            view = self.shard_view(self.master, p.name)
            if "norm" in p.name:
                view.fill_(1.0)
                continue
            g = torch.Generator(device=self.device)
            g.manual_seed(seed * 100003 + idx * 131 + self.rank)
            view.normal_(0.0, std, generator=g)
        self.publish_params()

    def publish_params(self) -> None:
        """master fp32 shard -> bf16 into every rank's replica (all-gather by push)."""
        if self.device.type != "cuda":
            for name, v in self.named_master_shards():
                i = self.layout.by_name[name]
                s = self.layout.segments[self.rank][i]
                self.params[s.full_offset: s.full_offset + s.numel].copy_(v.reshape(-1).to(torch.bfloat16))
            return
        lib = native.cuda()
        # publishing happens at start-up, after a checkpoint load and after an outer step, where ranks can be seconds
        # apart: meet on the host first so the bounded device barriers below only ever wait for kernel skew
        self.comm.host_barrier()
        self.comm.barrier()
        if self.reshard:      # no replica: each rank refreshes its own bf16 rows; peers fetch them when a block runs
            K.cast_to_bf16(self.master, self.param_shard[: self.master.numel()])
            self._root_fresh = False
            self._gbuf_holds = [-1, -1]
            self.comm.barrier()
            K.check_status(self.device)
            return
        for g, sa in enumerate(self._segs):
            if sa.n:
                check(lib.pb_zero_push_params(self._peer_params, self.world, self.rank, sa.n, sa.full, sa.shard, sa.numel,
                                              ptr(self.master), self.comm_ctas, stream_ptr()), "pb_zero_push_params")
        self.comm.barrier()
        K.check_status(self.device)   # a peer that never arrived: raise here rather than train on a partial replica

    # ------------------------------------------------------------------------------------------
    # workspace
    # ------------------------------------------------------------------------------------------
    def _buf(self, name: str, shape, dtype=torch.bfloat16) -> torch.Tensor:
        t = self._ws.get(name)
        n = math.prod(shape)
        if t is None or t.numel() < n or t.dtype != dtype:
            t = torch.empty(n, dtype=dtype, device=self.device)
            self._ws[name] = t
        return t[:n].view(shape)

    def _saved(self, layer: int, name: str, shape, dtype=torch.bfloat16) -> torch.Tensor:
        # with activation checkpointing only the block input is kept per layer
        key = f"L{layer}.{name}" if (not self._is_ckpt(layer) or name == "x") else f"Lshared.{name}"
        return self._buf(key, shape, dtype)

    def _is_ckpt(self, layer: int) -> bool:
        return self.ac_every > 0 and layer % self.ac_every == 0

    def default_seq_start(self, B: int, T: int) -> torch.Tensor:
        k = (B, T)
        if k not in self._seq_start_cache:
            self._seq_start_cache[k] = A.seq_start_from_batch(B, T, self.device)
        return self._seq_start_cache[k]

    # ------------------------------------------------------------------------------------------
    # forward / backward of one block
    # ------------------------------------------------------------------------------------------
    def _block_fwd(self, i: int, x: torch.Tensor, T: int, seq_start: torch.Tensor, out: torch.Tensor, recompute: bool = False) -> None:
        a = self.args
        M = x.shape[0]
        D, F, hd, H, KV = a.dim, a.hidden_dim, a.head_dim, a.n_heads, a.kv_heads
        pre = f"layers.{i}."
        fetch = self.reshard and not recompute      # a recompute inside the backward finds the block already gathered
        if fetch:
            self._fetch_block(i, whole=False)                   # normally started while the previous block ran
            if i + 1 < a.n_layers:
                self._fetch_block(i + 1, whole=False)           # the next block arrives under this one's kernels
            self._use_block(i)
        xn = self._saved(i, "xn", (M, D))
        rstd1 = self._saved(i, "rstd1", (M,), torch.float32)
        K.rmsnorm_fwd(x, self.w[pre + "attention_norm.weight"], a.norm_eps, out=xn, rstd=rstd1)
        qkv = self._saved(i, "qkv", (M, (H + 2 * KV) * hd))
        if fetch and not self._gbuf_whole[i % 2]:
            # all-gather fused into the first consuming GEMM: the other ranks' wq | wk | wv rows are pulled over NVLink by the
            # GEMM's own epilogue warps while its tensor cores work on the tiles whose rows have landed
            k2 = self._k2[1 + i]
            k2["calls"] += 1
            check(native.cuda().pb_gemm_bf16_allgather_parts(
                ptr(xn), k2["shards"], ptr(self.wqkv[i]), ptr(qkv), None, M, k2["n"], D, xn.stride(0), D, qkv.stride(0), 0, 0, 0,
                self.world, self.rank, 3, k2["rows"], k2["rpr"], k2["off"], ptr(k2["counters"]), k2["calls"], 0,
                ptr(K.status_word(self.device)), stream_ptr()), "pb_gemm_bf16_allgather_parts")
            self._gbuf_whole[i % 2] = True
            K.rope_(qkv, self._rope, T, H + KV, hd)
        else:
            K.gemm_rope(xn, self.wqkv[i], qkv, self._rope, T, H + KV, hd)     # rotary embedding in the GEMM epilogue
        o = self._saved(i, "o", (M, H * hd))
        _, lse2 = A.attention_fwd(qkv, seq_start, H, KV, hd, out=o)
        self._ws[f"L{i}.lse2" if not self._is_ckpt(i) else "Lshared.lse2"] = lse2
        h = self._saved(i, "h", (M, D))
        K.gemm(o, self.w[pre + "attention.wo.weight"], out=h, residual=x)
        hn = self._saved(i, "hn", (M, D))
        rstd2 = self._saved(i, "rstd2", (M,), torch.float32)
        K.rmsnorm_fwd(h, self.w[pre + "ffn_norm.weight"], a.norm_eps, out=hn, rstd=rstd2)
        h13 = self._saved(i, "h13", (M, 2 * F))
        act = self._saved(i, "act", (M, F))
        K.gemm_swiglu(hn, self.w13[i], h13, act)                          # SwiGLU in the GEMM epilogue
        K.gemm(act, self.w[pre + "feed_forward.w2.weight"], out=out, residual=h)
        if fetch:
            self._release_block(i)

    def _wgrad(self, dy: torch.Tensor, x: torch.Tensor, g: torch.Tensor) -> None:
        """g[N,K] (+)= dy[M,N]^T x[M,K]"""
        ws = self.wgrad_stream
        if ws is None or not dy.is_cuda:
            K.gemm(dy, x, out=g, residual=g if self._accum else None, a_mn=True, b_mn=True)
            return
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        ws.wait_event(ready)
        with torch.cuda.stream(ws):
            K.gemm(dy, x, out=g, residual=g if self._accum else None, a_mn=True, b_mn=True)
            done = torch.cuda.Event()
            done.record(ws)
        self._readers[dy.data_ptr()] = done
        self._readers[x.data_ptr()] = done

    def _before_write(self, *tensors: torch.Tensor) -> None:
        """The main stream is about to overwrite these tensors: wait for weight-gradient GEMMs that still read them."""
        if not self._readers:
            return
        main = torch.cuda.current_stream()
        for t in tensors:
            ev = self._readers.pop(t.data_ptr(), None)
            if ev is not None:
                main.wait_event(ev)

    def _wait_all_wgrads(self) -> None:
        if self.wgrad_stream is not None and self._readers:
            torch.cuda.current_stream().wait_stream(self.wgrad_stream)
            self._readers.clear()

    def _block_bwd(self, i: int, x: torch.Tensor, dout: torch.Tensor, T: int, seq_start: torch.Tensor, dx: torch.Tensor) -> None:
        a = self.args
        M = x.shape[0]
        D, F, hd, H, KV = a.dim, a.hidden_dim, a.head_dim, a.n_heads, a.kv_heads
        pre = f"layers.{i}."
        if self._is_ckpt(i):   # recompute the block's activations into the shared workspace
            self._wait_all_wgrads()    # weight gradients of the block above still read that workspace
            self._block_fwd(i, x, T, seq_start, self._buf("ckpt_out", (M, D)), recompute=True)
        sv = lambda n, shp, dt=torch.bfloat16: self._saved(i, n, shp, dt)  # noqa: E731
        xn, rstd1, qkv, o = sv("xn", (M, D)), sv("rstd1", (M,), torch.float32), sv("qkv", (M, (H + 2 * KV) * hd)), sv("o", (M, H * hd))
        lse2 = self._ws[f"L{i}.lse2" if not self._is_ckpt(i) else "Lshared.lse2"]
        h, hn, rstd2 = sv("h", (M, D)), sv("hn", (M, D)), sv("rstd2", (M,), torch.float32)
        h13, act = sv("h13", (M, 2 * F)), sv("act", (M, F))
        # out = h + act @ w2^T
        self._wgrad(dout, act, self.g[pre + "feed_forward.w2.weight"])
        # in place: h13 becomes d(h13); d(act) = dout @ w2 stays inside the GEMM whose epilogue does the SwiGLU backward
        self._before_write(h13)
        K.gemm_dswiglu(dout, self.w[pre + "feed_forward.w2.weight"], h13,
                       dact_ws=None if dout.is_cuda else self._buf("dact", (M, F)))
        dhn = self._buf("dhn", (M, D))
        K.gemm(h13, self.w13[i], out=dhn, b_mn=True)
        self._wgrad(h13, hn, self.g13[i])
        dh = self._buf("dh", (M, D))
        self._before_write(dh)
        K.rmsnorm_bwd(h, self.w[pre + "ffn_norm.weight"], rstd2, dhn, self.g[pre + "ffn_norm.weight"], dres=dout, dx=dh,
                      accumulate_dw=self._accum)
        # h = x + o @ wo^T
        do = self._buf("do", (M, H * hd))
        # dO = dh @ wo; the dO . O row sums of the attention backward come out of the same kernel where it applies
        dots = A.row_dots_buffer(dh.device, M, H) if dh.is_cuda else None
        if dots is None or not K.gemm_rowdot(dh, self.w[pre + "attention.wo.weight"], do, o, dots, hd, b_mn=True):
            K.gemm(dh, self.w[pre + "attention.wo.weight"], out=do, b_mn=True)
            dots = None
        self._wgrad(dh, o, self.g[pre + "attention.wo.weight"])
        dqkv = self._buf("dqkv", (M, (H + 2 * KV) * hd))
        self._before_write(dqkv)
        A.attention_bwd(qkv, o, do, lse2, seq_start, H, KV, hd, dqkv=dqkv, rope_table=self._rope, seq_len=T, row_dots=dots)
        dxn = self._buf("dxn", (M, D))
        K.gemm(dqkv, self.wqkv[i], out=dxn, b_mn=True)
        self._wgrad(dqkv, xn, self.gqkv[i])
        self._before_write(dx)
        K.rmsnorm_bwd(x, self.w[pre + "attention_norm.weight"], rstd1, dxn, self.g[pre + "attention_norm.weight"], dres=dh,
                      dx=dx, accumulate_dw=self._accum)
        if self._reduce_in_backward:
            self._reduce_group(1 + i, overlapped=True)     # this block's gradients are final: reduce them under the next block's backward

    # ------------------------------------------------------------------------------------------
    # full micro-step
    # ------------------------------------------------------------------------------------------
    def forward_backward(self, tokens: torch.Tensor, labels: torch.Tensor, seq_start: torch.Tensor | None = None,
                         loss_scale: float = 1.0, last_microbatch: bool = True) -> dict[str, torch.Tensor]:
        """One micro-batch: forward, loss, backward; gradients accumulate until ``optimizer_step``.
        Returns device scalars ``loss`` (mean CE over non-ignored tokens) and ``z_loss``."""
        a = self.args
        B, T = tokens.shape
        M = B * T
        D, V, L = a.dim, a.vocab_size, a.n_layers
        if seq_start is None:
            seq_start = self.default_seq_start(B, T)
        self._wait_all_wgrads()      # the forward overwrites the saved activations that the last weight gradients read
        if self.reshard:
            self.comm_stream.wait_stream(torch.cuda.current_stream())    # gathers start after everything before this call
            self._ensure_root()
        self._reduced_groups.clear()
        self._reduce_in_backward = bool(last_microbatch and self.overlap_reduce and self.device.type == "cuda")
        tok = tokens.reshape(-1)
        lab = labels.reshape(-1)
        xs = [self._buf(f"L{i}.x", (M, D)) for i in range(L + 1)]
        K.embedding_fwd(tok, self.w["tok_embeddings.weight"], out=xs[0])
        for i in range(L):
            self._block_fwd(i, xs[i], T, seq_start, xs[i + 1])
        # ---- head: final norm + chunked linear / cross-entropy / gradient ----
        hn = self._buf("head.hn", (M, D))
        rstd = self._buf("head.rstd", (M,), torch.float32)
        K.rmsnorm_fwd(xs[L], self.w["norm.weight"], a.norm_eps, out=hn, rstd=rstd)
        dhn = self._buf("head.dhn", (M, D))
        loss_rows = self._buf("head.loss_rows", (M,), torch.float32)
        z_rows = self._buf("head.z_rows", (M,), torch.float32)
        inv = K.count_valid(lab)
        Vp = (V + 7) // 8 * 8
        Mc = min(self.ce_chunk, M)
        logits_buf = self._buf("head.logits", (Mc, Vp))
        Wout, gWout = self.w["output.weight"], self.g["output.weight"]
        accum_head = self._accum
        for c0 in range(0, M, Mc):
            c1 = min(M, c0 + Mc)
            lg = logits_buf[: c1 - c0, :V]
            K.gemm(hn[c0:c1], Wout, out=lg)
            K.cross_entropy_(lg, lab[c0:c1], inv, loss_rows[c0:c1], z_rows[c0:c1], grad_scale=loss_scale,
                             z_mode=self.z_mode, z_weight=self.z_weight)
            K.gemm(lg, Wout, out=dhn[c0:c1], b_mn=True)
            K.gemm(lg, hn[c0:c1], out=gWout, residual=gWout if accum_head else None, a_mn=True, b_mn=True)
            accum_head = True
        out = self._buf("head.scalars", (2,), torch.float32)
        K.sum_f32(loss_rows, out[0:1], scale_ptr=inv[0:1])
        K.sum_f32(z_rows, out[1:2], scale_ptr=inv[0:1], scale=self.z_weight)
        dx = self._buf("dx_a", (M, D))
        K.rmsnorm_bwd(xs[L], self.w["norm.weight"], rstd, dhn, self.g["norm.weight"], dx=dx, accumulate_dw=self._accum)
        if self._reduce_in_backward:
            self._reduce_group(L + 1, overlapped=True)     # head group (final norm + output projection)
        # ---- blocks in reverse ----
        other = self._buf("dx_b", (M, D))
        for i in reversed(range(L)):
            if self.reshard:       # re-gather, one block ahead of the backward
                self._fetch_block(i, whole=True)
                if i > 0:
                    self._fetch_block(i - 1, whole=True)
                self._use_block(i)
            self._block_bwd(i, xs[i], dx, T, seq_start, other)
            if self.reshard:
                self._release_block(i)
            dx, other = other, dx
        # ---- embedding ----
        gE = self.g["tok_embeddings.weight"]
        if not self._accum:
            gE.zero_()
        K.embedding_bwd(tok, dx, gE)
        self._reduce_in_backward = False
        self._accum = True
        return {"loss": out[0], "z_loss": out[1]}

    # ------------------------------------------------------------------------------------------
    # optimizer
    # ------------------------------------------------------------------------------------------
    def optimizer_step(self, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1,
                       max_norm: float = 1.0) -> torch.Tensor:
        """Reduce-scatter + global-norm clip + sharded AdamW + all-gather. Returns the (device
        scalar) total gradient norm before clipping."""
        assert self._accum, "optimizer_step without gradients"
        self.opt_step += 1
        if self.device.type != "cuda":
            return self._optimizer_step_cpu(lr, betas, eps, weight_decay, max_norm)
        lib = native.cuda()
        W = self.world
        # Reduce-scatter by pull, one launch per parameter group. Groups whose gradients were final during the backward are
        # already in flight on the comm stream (each behind its own peer barrier); the rest (the embedding, or everything
        # when the overlap is off) follow now. The sum of squares is kept per group and added up in group order, so the
        # overlapped and the serial schedule produce the same bits.
        for g in range(len(self._segs)):
            if g not in self._reduced_groups:
                self._reduce_group(g, overlapped=self.overlap_reduce)
        if self.overlap_reduce:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        self._reduced_groups.clear()
        K.sum_f32(self._norm_parts, self._norm_local[0:1])
        self.comm.allreduce_scalars(self._norm_local, self._norm_global, 1)   # also orders: all ranks done reading grads
        if self._shard_opt is not None:
            assert not self.reshard, "a shard optimizer needs the resident replica (publish_params refreshes it)"
            self._shard_optimizer_update(lr, max_norm)
            self._accum = False
            return self._norm_global[0].sqrt()
        if self.reshard:
            # no replica to refresh: the new bf16 values go to this rank's own rows only (a one-rank "push")
            n = self.master.numel()
            one = (C.c_longlong * 1)
            check(lib.pb_zero_adamw_gather((C.c_void_p * 1)(self.param_shard.data_ptr()), 1, 0, 1, one(0), one(0), one(n), ptr(self.master),
                                           ptr(self.grad_shard), ptr(self.exp_avg), ptr(self.exp_avg_sq), lr, betas[0], betas[1],
                                           eps, weight_decay, self.opt_step, ptr(self._norm_global), max_norm,
                                           min(self.comm_ctas * 4, 1024), stream_ptr()), "pb_zero_adamw_gather")
            self._root_fresh = False
            self._gbuf_holds = [-1, -1]
        for g, sa in enumerate(self._segs_step if not self.reshard else []):
            if sa.n == 0:
                continue
            check(lib.pb_zero_adamw_gather(self._peer_params, W, self.rank, sa.n, sa.full, sa.shard, sa.numel, ptr(self.master),
                                           ptr(self.grad_shard), ptr(self.exp_avg), ptr(self.exp_avg_sq), lr, betas[0], betas[1],
                                           eps, weight_decay, self.opt_step, ptr(self._norm_global), max_norm,
                                           self._opt_ctas(sa), stream_ptr()), "pb_zero_adamw_gather")
        self.comm.barrier()                                   # every rank's replica is complete
        self._accum = False
        return self._norm_global[0].sqrt()

    def _reduce_group(self, g: int, overlapped: bool) -> None:
        """Reduce-scatter (+ cast / scale + sum of squares) of parameter group ``g``: after a peer barrier that says every
        rank has written its gradients of the group, pull this rank's slices from all ranks. ``overlapped``: on the comm
        stream, behind an event of the main stream, so it runs under whatever the main stream does next."""
        sa = self._segs[g]
        self._reduced_groups.add(g)
        lib = native.cuda()
        main = torch.cuda.current_stream()
        stream = self.comm_stream if overlapped else main
        if overlapped:
            ev = torch.cuda.Event()
            ev.record(main)
            stream.wait_event(ev)
        if self.wgrad_stream is not None:
            stream.wait_stream(self.wgrad_stream)      # the group's weight gradients are produced there
        self.comm.barrier(slot=4, stream=stream)
        if sa.n == 0:
            with torch.cuda.stream(stream):
                self._norm_parts[g:g + 1].zero_()
            return
        check(lib.pb_zero_reduce_grads(self._peer_grads, self.world, self.rank, int(self.grad_dtype == torch.float32), sa.n, sa.full,
                                       sa.shard, sa.numel, ptr(self.grad_shard), 1.0 / self.world, ptr(self._partials),
                                       ptr(self._norm_parts[g:g + 1]), 0, self._opt_ctas(sa), stream_ptr(stream)),
              "pb_zero_reduce_grads")

    def _opt_ctas(self, sa) -> int:
        """Grid of the reduce and AdamW launches. One merged segment streams best from a grid of one CTA per SM
        slot; a table of many segments (sharded runs) needs enough CTAs for the per-segment split to follow the
        segment sizes: one CTA per 32k elements, within the size of the partial-sum scratch."""
        base = min(self.comm_ctas * 4, 1024)
        if sa.n <= 1:
            return base
        return int(max(base, sa.n, min(sa.total // 32768, self._partials.numel())))

    def _optimizer_step_cpu(self, lr, betas, eps, weight_decay, max_norm) -> torch.Tensor:
        """Single-rank CPU twin of the update (same math through the CPU branches of the ops)."""
        assert self.world == 1
        for s in self.layout.segments[0]:
            self.grad_shard[s.shard_offset: s.shard_offset + s.numel].copy_(self.grads[s.full_offset: s.full_offset + s.numel])
        K.sumsq(self.grad_shard, self._norm_global[0:1])
        norm = self._norm_global[0].sqrt()
        if self._shard_opt is not None:
            norm = norm.clone()
            self._shard_optimizer_update(lr, max_norm)
            self._accum = False
            return norm
        K.adamw_(self.master, self.grad_shard, self.exp_avg, self.exp_avg_sq, None, lr, betas[0], betas[1], eps, weight_decay,
                 self.opt_step, gnorm=norm if max_norm > 0 else None, max_norm=max_norm)
        self.publish_params()
        self._accum = False
        return norm

    def zero_grad(self) -> None:
        self._accum = False

    def train_step(self, tokens: torch.Tensor, labels: torch.Tensor, lr: float, micro_bs: int | None = None,
                   betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1, max_norm: float = 1.0,
                   seq_start: torch.Tensor | None = None, sync_loss: bool = True):
        """One optimizer step on this rank's batch ``[B, T]`` (host or device tensors).

        Host tensors (pinned recommended) are copied to the device on the compute stream; the batch
        is split into micro-batches of ``micro_bs`` sequences whose gradients accumulate; then the
        reduce-scatter / clip / AdamW / all-gather update runs. Returns ``(loss, grad_norm)`` as
        Python floats when ``sync_loss`` (one device-to-host read), else as device scalars."""
        B = tokens.shape[0]
        micro_bs = micro_bs or B
        assert B % micro_bs == 0
        n_micro = B // micro_bs
        if not tokens.is_cuda and self.device.type == "cuda":
            tokens = tokens.to(self.device, non_blocking=True)
            labels = labels.to(self.device, non_blocking=True)
        total = self._buf("step.loss", (2,), torch.float32)
        total.zero_()
        for mb in range(n_micro):
            sl = slice(mb * micro_bs, (mb + 1) * micro_bs)
            ss = None
            if seq_start is not None:
                T = tokens.shape[1]
                ss = seq_start[mb * micro_bs * T: (mb + 1) * micro_bs * T] - mb * micro_bs * T
            out = self.forward_backward(tokens[sl], labels[sl], seq_start=ss, loss_scale=1.0 / n_micro,
                                        last_microbatch=(mb == n_micro - 1))
            total[0] += out["loss"] / n_micro
            total[1] += out["z_loss"] / n_micro
        norm = self.optimizer_step(lr, betas, eps, weight_decay, max_norm)
        if sync_loss:
            # the step's only device->host read; the device status word rides along, so a peer wait that gave up
            # (PB_ERR_TIMEOUT_PEER) surfaces as an exception of this step instead of a silently partial update
            st = K.status_word(self.device) if self.device.type == "cuda" else None
            vals = [total[0], total[1], norm] + ([st[0].to(torch.float32)] if st is not None else [])
            host = torch.stack(vals).tolist()
            if st is not None and host[3] != 0.0:
                code = int(host[3])
                st.zero_()
                raise native.NativeError(f"train_step: device kernel reported error code {code & 0xff} (peer/cta {code >> 8}); "
                                         "the update of this step is not valid")
            return host[0], host[2]
        return total[0], norm

    # ------------------------------------------------------------------------------------------
    # inference-style forward (logits), used by tests and evaluation
    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_logits(self, tokens: torch.Tensor, seq_start: torch.Tensor | None = None) -> torch.Tensor:
        a = self.args
        B, T = tokens.shape
        M = B * T
        if seq_start is None:
            seq_start = self.default_seq_start(B, T)
        if self.reshard:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            self._ensure_root()
        x = self._buf("L0.x", (M, a.dim))
        K.embedding_fwd(tokens.reshape(-1), self.w["tok_embeddings.weight"], out=x)
        for i in range(a.n_layers):
            nxt = self._buf(f"L{i + 1}.x", (M, a.dim))
            self._block_fwd(i, x, T, seq_start, nxt)
            x = nxt
        hn, _ = K.rmsnorm_fwd(x, self.w["norm.weight"], a.norm_eps)
        return K.gemm(hn, self.w["output.weight"], out_dtype=torch.float32).reshape(B, T, -1)
