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
