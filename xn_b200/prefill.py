"""Column-parallel prefill of the fp8 linears over the GPUs of one box.

The reference has no multi-GPU path; this is the partitioning the benchmark's decoder configuration
describes: every rank holds the full activations x [M, K] and the rows [r*N/W, (r+1)*N/W) of each
(out, in) weight, computes its slice of y = x W^T and the slices are assembled on every rank.

Two assembly routes:
  "peer"   the GEMM epilogue stores each finished tile straight into every rank's [M, N] output
           (symmetric memory; xn_mm_linear_fp8_pieces_scatter): transfer and tensor-core work overlap tile
           by tile, no staging buffer, no re-layout pass.  With an NVLink multicast mapping of the output
           (NVSwitch) each 16-byte piece is ONE multimem.st that the switch replicates to every rank
           (xn_mm_linear_fp8_pieces_multicast); otherwise one plain store per peer;
  "gather" local GEMM, then torch.distributed all_gather_into_tensor and a re-layout
           ([W, M, N/W] -> [M, N]); works with any backend (the CPU tests run it on gloo) and is the
           baseline the peer route is timed against.

For the gated FFN rank r owns the matching gate and up channels, [r*h/W, (r+1)*h/W) of each half, so
silu(gate)*up is local and only [M, h] (not [M, 2h]) has to be assembled.

Run `python -m torch.distributed.run --nproc-per-node W -m xn_b200.prefill` for a self-check + timing.
"""
from __future__ import annotations

import json
import os
import sys


def shard_rows(n: int, world: int, rank: int, align: int = 16):
    """[start, stop) of the output channels rank owns: equal blocks of ceil(n/world) rounded up to
    `align` channels (the last ranks may own fewer, possibly none)."""
    per = -(-n // world)
    per = -(-per // align) * align
    start = min(n, rank * per)
    return start, min(n, start + per)


def gated_shard_rows(hidden: int, world: int, rank: int, align: int = 16):
    """Rows of a [2*hidden, K] gated-FFN weight owned by rank: the same channel range of both halves."""
    a, b = shard_rows(hidden, world, rank, align)
    return (a, b), (hidden + a, hidden + b)


def assemble_columns(staged, world: int, n: int, align: int = 16):
    """[W, M, per] gathered slices -> [M, n]: slice r supplies columns shard_rows(n, W, r)."""
    import torch
    m = staged.shape[1]
    out = torch.empty(m, n, dtype=staged.dtype, device=staged.device)
    for r in range(world):
        a, b = shard_rows(n, world, r, align)
        if b > a:
            out[:, a:b] = staged[r, :, : b - a]
    return out


def column_parallel_gather(x, local_linear, n: int, group=None, align: int = 16):
    """The "gather" route with a pluggable local linear: local_linear(x, start, stop) -> [M, stop-start]."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    a, b = shard_rows(n, world, rank, align)
    per = shard_rows(n, world, 0, align)[1]
    m = x.shape[0]
    local = torch.zeros(m, per, dtype=torch.bfloat16 if x.dtype != torch.float32 else x.dtype, device=x.device)
    if b > a:
        y = local_linear(x, a, b)
        local = local.to(y.dtype)
        local[:, : b - a] = y
    staged = torch.empty(world, m, per, dtype=local.dtype, device=x.device)
    dist.all_gather_into_tensor(staged.view(world * m, per), local, group=group)
    return assemble_columns(staged, world, n, align)


class PeerPrefillLinear:
    """One fp8 linear, column-split, results assembled by epilogue stores into peer memory."""

    def __init__(self, wq, ws, n: int, k: int, m_max: int, group=None, multicast: bool = True):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n, self.k = n, k
        self.a, self.b = shard_rows(n, self.world, self.rank)
        self.wq, self.ws = wq[self.a:self.b].contiguous(), ws[self.a:self.b].contiguous()
        self.out = symm.empty(m_max, n, dtype=torch.bfloat16, device=wq.device)
        self.hdl = symm.rendezvous(self.out, group=dist.group.WORLD if group is None else group)
        import ctypes as C
        self.ptrs = (C.c_void_p * self.world)(*[int(p) for p in self.hdl.buffer_ptrs])
        # NVLink multicast mapping of the same buffers, when the fabric offers one (NVSwitch): one store reaches
        # every rank.  Usable when every rank's slice keeps the 16-byte store granularity.
        self.mc_ptr = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        self.multicast = bool(self.mc_ptr) and multicast and n % 8 == 0 and self.a % 8 == 0 and (self.b - self.a) % 8 == 0

    def forward(self, hi, lo, xs, m: int):
        import torch

        from ._lib import check, lib
        if self.b > self.a and self.multicast:
            check(lib().xn_mm_linear_fp8_pieces_multicast(self.mc_ptr, self.n, self.a, hi.data_ptr(),
                                                          lo.data_ptr() if lo is not None else None, xs.data_ptr(),
                                                          self.wq.data_ptr(), self.ws.data_ptr(), m, self.b - self.a, self.k,
                                                          torch.cuda.current_stream().cuda_stream))
        elif self.b > self.a:
            check(lib().xn_mm_linear_fp8_pieces_scatter(self.ptrs, self.world, self.n, self.a, hi.data_ptr(),
                                                        lo.data_ptr() if lo is not None else None, xs.data_ptr(),
                                                        self.wq.data_ptr(), self.ws.data_ptr(), m, self.b - self.a, self.k,
                                                        torch.cuda.current_stream().cuda_stream))
        self.hdl.barrier()  # every rank's slices have landed everywhere
        return self.out[:m]


class _Gathered:
    """A [rows, cols] bf16 buffer that every rank holds in full and each rank fills its column slice of -- in every
    rank's copy at once: symmetric memory with the peers' pointers (plain stores) and, where the fabric offers it,
    an NVLink multicast mapping (one multimem.st per 16 bytes).  With one rank it is an ordinary tensor."""

    def __init__(self, rows: int, cols: int, device, world: int, group, multicast: bool):
        import ctypes as C

        import torch
        self.world = world
        if world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm
            self.t = symm.empty(rows, cols, dtype=torch.bfloat16, device=device)
            self.hdl = symm.rendezvous(self.t, group=dist.group.WORLD if group is None else group)
            ptrs = [int(p) for p in self.hdl.buffer_ptrs]
            self.mc_ptr = int(getattr(self.hdl, "multicast_ptr", 0) or 0) if multicast else 0
        else:
            self.t = torch.empty(rows, cols, dtype=torch.bfloat16, device=device)
            self.hdl, ptrs, self.mc_ptr = None, [self.t.data_ptr()], 0
        self.ptrs = (C.c_void_p * len(ptrs))(*ptrs)
        self.mc = (C.c_void_p * 1)(self.mc_ptr)

    def barrier(self):
        if self.hdl is not None:
            self.hdl.barrier()


class PrefillStack:
    """A T-token prefill of one stream through the decoder stack of xn_b200/decoder.py (pre-norm, fused qkv, causal
    attention, gated SiLU FFN, fp8-e4m3 weights, no rope) with every weight split by output channel over the ranks
    -- the tensor-parallel layout of the benchmark's prefill configuration:

      in_proj     rank r owns the q, k and v rows of its heads [r*H/W, (r+1)*H/W): its slice of the projection is
                  all its attention needs, so nothing is exchanged here
      attention   causal, per head, local: q.k^T (batched tcgen05 GEMM over a zero-copy view of the slice) ->
                  scale / mask / softmax in one pass -> p.v (batched GEMM with the [ctx, 128] right-hand side read as
                  an MN-major operand); the [T, d/W] result is written into every rank's [T, d] buffer
      out_proj    rows [r*d/W, ...): the GEMM epilogue stores its tiles into every rank's [T, d] buffer
      linear_in   the gate rows and the up rows of channels [r*h/W, ...) (xn-moshi/src/transformer.rs:239-245: gate =
                  first h output channels, up = second h), so silu(gate)*up is local and [T, h/W] -- not [T, 2h/W]
                  -- is written into every rank's [T, h] buffer
      linear_out  rows [r*d/W, ...), epilogue stores as for out_proj
    Four exchanges per layer, 2*T*(3d + h) bytes in total, each followed by a symmetric-memory barrier.  Every
    output element is accumulated over k in the same order whatever the split, so the result is bit-identical to
    the one-rank run (`single=True` builds that run inside a multi-rank job, for the comparison).  All ranks draw the
    same weights from the seed and keep their slices."""

    def __init__(self, n_layers: int, d_model: int, n_heads: int, ffn_hidden: int, tokens: int, device, group=None,
                 eps: float = 1e-5, seed: int = 4, variant: int = 0, multicast: bool = True, single: bool = False,
                 fused_attention: bool = True):
        import torch

        from .ops import quantize_weights_fp8
        self.fused_attention = fused_attention
        if not single and (group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized())):
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        W, r = self.world, self.rank
        assert d_model == n_heads * 128 and n_heads % W == 0 and (ffn_hidden // W) % 16 == 0 and ffn_hidden % W == 0
        self.L, self.d, self.H, self.hid, self.T = n_layers, d_model, n_heads, ffn_hidden, tokens
        self.dl, self.hl, self.Hl = d_model // W, ffn_hidden // W, n_heads // W
        self.eps, self.variant, self.dev = eps, variant, device
        d, hid, dl, hl = d_model, ffn_hidden, self.dl, self.hl
        g = torch.Generator(device=device).manual_seed(seed)

        def qrows(n, k, ranges):
            w = torch.randn(n, k, generator=g, device=device) * 0.02
            q, s = quantize_weights_fp8(w)  # per-channel scales: a row's code does not depend on the other rows
            del w
            idx = torch.cat([torch.arange(a, b, device=device) for a, b in ranges])
            return q[idx].contiguous(), s[idx].contiguous()

        self.layers = []
        for _ in range(n_layers):
            self.layers.append({
                "norm1": torch.ones(d, device=device, dtype=torch.bfloat16),
                "norm2": torch.ones(d, device=device, dtype=torch.bfloat16),
                "in_proj": qrows(3 * d, d, [(j * d + r * dl, j * d + (r + 1) * dl) for j in range(3)]),
                "out_proj": qrows(d, d, [(r * dl, (r + 1) * dl)]),
                "linear_in": qrows(2 * hid, d, [(r * hl, (r + 1) * hl), (hid + r * hl, hid + (r + 1) * hl)]),
                "linear_out": qrows(d, hid, [(r * dl, (r + 1) * dl)]),
            })
        T = tokens
        u8 = dict(dtype=torch.uint8, device=device)
        bf = dict(dtype=torch.bfloat16, device=device)
        kmax = max(d, hid)
        self.hi, self.lo = torch.empty(T * kmax, **u8), torch.empty(T * kmax, **u8)
        self.xs = torch.empty(T, dtype=torch.float32, device=device)
        self.qkv = torch.empty(T, 3 * dl, **bf)
        if fused_attention:
            self.attn_rows = torch.empty(T, dl, **bf)  # heads side by side in a row, as the out projection reads them
        else:
            self.scores = torch.empty(self.Hl, T, T, **bf)
            self.attn_l = torch.empty(self.Hl, T, 128, **bf)
        self.h_l = torch.empty(T, 2 * hl, **bf)
        self.g_l = torch.empty(T, hl, **bf)
        self.x_mid = torch.empty(T, d, **bf)
        self.x_out = torch.empty(T, d, **bf)
        self.attn_full = _Gathered(T, d, device, W, group, multicast)
        self.proj_full = _Gathered(T, d, device, W, group, multicast)
        self.gated_full = _Gathered(T, hid, device, W, group, multicast)

    # -- helpers -------------------------------------------------------------------------------
    def _s(self):
        import torch
        return torch.cuda.current_stream().cuda_stream

    def _lo(self):
        return self.lo.data_ptr() if self.variant == 0 else None

    def _linear_local(self, y, wq_ws, n, k):
        from ._lib import check, lib
        wq, ws = wq_ws
        check(lib().xn_mm_linear_fp8_pieces(y.data_ptr(), self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), wq.data_ptr(),
                                            ws.data_ptr(), self.T, n, k, self._s()))

    def _linear_gathered(self, dst: _Gathered, wq_ws, n_total, k):
        """Column-parallel linear whose epilogue writes this rank's [T, n_total / W] slice into every rank's buffer."""
        from ._lib import check, lib
        wq, ws = wq_ws
        nl = n_total // self.world
        if dst.mc_ptr:
            check(lib().xn_mm_linear_fp8_pieces_multicast(dst.mc_ptr, n_total, self.rank * nl, self.hi.data_ptr(), self._lo(),
                                                          self.xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), self.T, nl, k,
                                                          self._s()))
        else:
            check(lib().xn_mm_linear_fp8_pieces_scatter(dst.ptrs, self.world, n_total, self.rank * nl, self.hi.data_ptr(),
                                                        self._lo(), self.xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), self.T,
                                                        nl, k, self._s()))
        dst.barrier()

    def _gather(self, dst: _Gathered, src, n_total, groups):
        from ._lib import check, lib
        nl = n_total // self.world
        if dst.mc_ptr:
            check(lib().xn_mm_scatter_columns(dst.mc, 1, 1, 2 * n_total, 2 * self.rank * nl, src.data_ptr(), self.T, 2 * nl,
                                              groups, self._s()))
        else:
            check(lib().xn_mm_scatter_columns(dst.ptrs, self.world, 0, 2 * n_total, 2 * self.rank * nl, src.data_ptr(), self.T,
                                              2 * nl, groups, self._s()))
        dst.barrier()

    def forward(self, x):
        """x: [tokens, d_model] bf16, the same on every rank.  Returns the stack's [tokens, d_model] output (on every rank)."""
        import math

        from ._lib import BF16, check, lib
        from .ops import attention_prefill_, matmul_causal_
        L, T, d, hid, dl, hl, Hl = lib(), self.T, self.d, self.hid, self.dl, self.hl, self.Hl
        s = self._s()
        cur = x
        for li, lay in enumerate(self.layers):
            if li == 0:
                check(L.xn_mm_rms_norm_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), None, cur.data_ptr(),
                                                  lay["norm1"].data_ptr(), BF16, T, d, self.eps, s))
            self._linear_local(self.qkv, lay["in_proj"], 3 * dl, d)
            qkv4 = self.qkv.view(T, 3, Hl, 128)
            q, k, v = (qkv4[:, j].transpose(0, 1) for j in range(3))      # [Hl, T, 128] views, rows 3*dl apart
            if self.fused_attention:
                # one kernel for the rank's heads: scores and probabilities never leave the SM (a single rank owns
                # every head and writes the rows the out projection reads: nothing to exchange)
                attention_prefill_(self.attn_full.t if self.world == 1 else self.attn_rows, q, k, v, 1.0 / math.sqrt(128.0))
            else:
                # q.k^T, one launch for the rank's heads; tiles beyond the causal horizon are skipped
                matmul_causal_(self.scores, q, k, True, 1, 0)
                check(L.xn_mm_softmax_causal(BF16, self.scores.data_ptr(), self.scores.data_ptr(), Hl, T, T,
                                             1.0 / math.sqrt(128.0), 0, s))
                # p.v, [T, 128] right-hand side per head; every row tile stops at its horizon
                matmul_causal_(self.attn_l, self.scores, v, False, 2, 0)
            if self.fused_attention:
                if self.world > 1:
                    self._gather(self.attn_full, self.attn_rows, d, 1)
            else:
                self._gather(self.attn_full, self.attn_l, d, Hl)
            check(L.xn_mm_split_rows_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), self.attn_full.t.data_ptr(), BF16,
                                          T, d, s))
            self._linear_gathered(self.proj_full, lay["out_proj"], d, d)
            check(L.xn_mm_add_rms_norm_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), self.x_mid.data_ptr(),
                                                  cur.data_ptr(), self.proj_full.t.data_ptr(), lay["norm2"].data_ptr(), BF16, T,
                                                  d, self.eps, s))
            self._linear_local(self.h_l, lay["linear_in"], 2 * hl, d)
            if self.world == 1:
                # a single rank holds whole rows of the gated activations: gate and split in one kernel
                check(L.xn_mm_silu_mul_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), self.h_l.data_ptr(), BF16, T,
                                                  hl, s))
            else:
                check(L.xn_mm_silu_mul(BF16, self.g_l.data_ptr(), self.h_l.data_ptr(), T, hl, s))
                self._gather(self.gated_full, self.g_l, hid, 1)
                check(L.xn_mm_split_rows_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), self.gated_full.t.data_ptr(),
                                              BF16, T, hid, s))
            self._linear_gathered(self.proj_full, lay["linear_out"], d, hid)
            if li + 1 < len(self.layers):
                check(L.xn_mm_add_rms_norm_split_e4m3(self.hi.data_ptr(), self._lo(), self.xs.data_ptr(), self.x_out.data_ptr(),
                                                      self.x_mid.data_ptr(), self.proj_full.t.data_ptr(),
                                                      self.layers[li + 1]["norm1"].data_ptr(), BF16, T, d, self.eps, s))
            else:
                check(L.xn_mm_add(BF16, self.x_out.data_ptr(), self.x_mid.data_ptr(), self.proj_full.t.data_ptr(), T * d, s))
            cur = self.x_out
        return self.x_out

    def flops(self) -> float:
        """Useful floating-point operations of one forward pass over all ranks (linears + causal attention)."""
        d, hid, T = self.d, self.hid, self.T
        lin = 2.0 * T * (3 * d * d + d * d + 2 * hid * d + d * hid)
        att = 2.0 * 2.0 * self.H * T * T * 128 / 2.0   # q.k^T and p.v, half of the square is visible
        return self.L * (lin + att)

    def exchanged_bytes_per_rank(self) -> int:
        """Bytes each rank delivers to its peers per forward pass."""
        return self.L * 2 * self.T * (3 * self.dl + self.hl) * (self.world - 1)


def _main():
    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import xn_b200 as xn
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    m = int(os.environ.get("XN_PREFILL_M", "4096"))
    shapes = [(12288, 4096, "qkv"), (4096, 4096, "out_proj"), (22528, 4096, "ffn_up"), (4096, 11264, "ffn_down")]
    report = []
    for n, k, name in shapes:
        g = torch.Generator(device=dev).manual_seed(4)  # same weights and inputs on every rank
        w = torch.randn(n, k, generator=g, device=dev) * 0.02
        wq, ws = xn.quantize_weights_fp8(w)
        del w
        x = torch.randn(m, k, generator=g, device=dev).bfloat16()
        hi, lo, xs = xn.split_rows_e4m3(x)
        full = xn.linear_fp8(x, wq, ws, 0)  # single-GPU result of the whole linear
        lin = PeerPrefillLinear(wq, ws, n, k, m)
        y = lin.forward(hi, lo, xs, m)
        torch.cuda.synchronize()
        same_peer = bool(torch.equal(y, full))

        def local_linear(xx, a, b):
            out = torch.empty(m, b - a, dtype=torch.bfloat16, device=dev)
            xn._lib.check(xn.lib().xn_mm_linear_fp8_pieces(out.data_ptr(), hi.data_ptr(), lo.data_ptr(), xs.data_ptr(),
                                                           wq[a:b].contiguous().data_ptr(), ws[a:b].contiguous().data_ptr(),
                                                           m, b - a, k, torch.cuda.current_stream().cuda_stream))
            return out
        y2 = column_parallel_gather(x, local_linear, n)
        same_gather = bool(torch.equal(y2, full))

        def timeit(fn, iters=10):
            for _ in range(3):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        wl = wq[lin.a:lin.b].contiguous()
        wsl = ws[lin.a:lin.b].contiguous()
        out_l = torch.empty(m, max(1, lin.b - lin.a), dtype=torch.bfloat16, device=dev)
        t_peer = timeit(lambda: lin.forward(hi, lo, xs, m))
        t_gather = timeit(lambda: column_parallel_gather(x, local_linear, n))
        t_local = timeit(lambda: xn._lib.check(xn.lib().xn_mm_linear_fp8_pieces(
            out_l.data_ptr(), hi.data_ptr(), lo.data_ptr(), xs.data_ptr(), wl.data_ptr(), wsl.data_ptr(), m,
            lin.b - lin.a, k, torch.cuda.current_stream().cuda_stream)))
        t_full = timeit(lambda: xn.linear_fp8(x, wq, ws, 0))
        report.append({"name": name, "m": m, "n": n, "k": k, "world": world, "identical_peer": same_peer,
                       "identical_gather": same_gather, "ms_peer_fused": t_peer, "ms_nccl_gather": t_gather,
                       "ms_local_gemm_only": t_local, "ms_one_gpu_full": t_full,
                       "nvlink_bytes_out_per_rank": 2 * m * (lin.b - lin.a) * (world - 1)})
        del lin
    if rank == 0:
        print(json.dumps({"prefill_column_parallel": report}), flush=True)
    ok = all(r["identical_peer"] and r["identical_gather"] for r in report)
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    _main()
