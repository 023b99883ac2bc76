"""CPU: host-side logic of the column-parallel prefill with two gloo ranks.  The local linear is the
oracle (there is no CPU product path); what is under test is the sharding arithmetic, the gated-FFN
pairing and the gather + re-layout, which the GPU path shares."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, k, m, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import oracle
    from xn_b200_prefill_shim import prefill  # noqa: F401  (loaded by path: the package needs the CUDA library)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    xb = oracle.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    wq, ws = oracle.quantize_fp8_channel(w)

    def local_linear(x, a, b):
        y16, _ = oracle.linear_fp8(xb, wq[a:b], ws[a:b], 0)
        return torch.from_numpy(y16.view(np.int16)).view(torch.bfloat16)

    y = prefill.column_parallel_gather(torch.zeros(m, k, dtype=torch.bfloat16), local_linear, n)
    full16, _ = oracle.linear_fp8(xb, wq, ws, 0)
    ok = np.array_equal(y.view(torch.int16).numpy().view(np.uint16), full16)
    q.put((rank, bool(ok)))
    dist.destroy_process_group()


def _load_prefill():
    import importlib.util
    import sys
    import types
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("xn_b200_prefill", os.path.join(root, "xn_b200", "prefill.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    shim = types.ModuleType("xn_b200_prefill_shim")
    shim.prefill = mod
    sys.modules["xn_b200_prefill_shim"] = shim
    return mod


def test_shard_arithmetic():
    p = _load_prefill()
    for n, world in [(12288, 8), (4096, 8), (22528, 8), (4096, 3), (100, 8), (16, 8), (11264, 8)]:
        cover = []
        for r in range(world):
            a, b = p.shard_rows(n, world, r)
            assert 0 <= a <= b <= n and (a % 16 == 0 or a == n)
            cover += list(range(a, b))
        assert cover == list(range(n)), (n, world)
    (g0, g1), (u0, u1) = p.gated_shard_rows(11264, 8, 3)
    assert (g0, g1) == (4224, 5632) and (u0, u1) == (11264 + 4224, 11264 + 5632)
    staged = torch.arange(2 * 3 * 8, dtype=torch.float32).reshape(2, 3, 8)
    out = p.assemble_columns(staged, 2, 12, align=8)
    assert torch.equal(out[:, :8], staged[0]) and torch.equal(out[:, 8:], staged[1][:, :4])


def test_column_parallel_gather_two_gloo_ranks():
    _load_prefill()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_entry, args=(r, 2, port, 200, 256, 5, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    assert res == [(0, True), (1, True)]


def _worker_entry(rank, world, port, n, k, m, q):
    _load_prefill()
    _worker(rank, world, port, n, k, m, q)
