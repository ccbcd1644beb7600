"""Exchange + merge of KV-sequence shard partials over peer memory (fr_xchg_merge).

On one GPU the protocol runs for R emulated ranks as ONE cooperative launch (fr_xchg_selftest: same device code, grid row =
rank), several steps on the same buffers, against the merge rule evaluated in torch.  With two or more GPUs the real entry
runs in one process per GPU (buffers mapped through CUDA IPC, handles carried by gloo) and every rank's output is compared
with the merge of the gathered partials.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def make_parts(R, rows, g, empty=()):
    parts = []
    for r in range(R):
        p = torch.randn(rows, 130, generator=g)
        p[:, 128] = torch.randn(rows, generator=g) * 6                 # m in log2 units
        p[:, 129] = torch.rand(rows, generator=g) * 50 + 0.1           # l
        if r in empty:
            p[:, 128], p[:, 129] = float("-inf"), 0.0
        parts.append(p)
    return parts


@pytest.mark.parametrize("R,rows", [(2, 32), (4, 33), (8, 32), (3, 7), (8, 256), (1, 32)])
def test_emulated_ranks_one_launch(R, rows):
    from flagrot_releaser_b200 import kernels as K
    g = torch.Generator().manual_seed(100 * R + rows)
    bufs = None
    for step in range(5):
        parts = make_parts(R, rows, g, empty=(1,) if step == 2 and R > 1 else ())
        dparts = [p.cuda() for p in parts]
        outs = [torch.full((rows, 128), float("nan"), device="cuda") for _ in range(R)]
        if bufs is None:
            rc, bufs = K.xchg_selftest(dparts, outs)
        else:
            rc = K.xchg_selftest_step(dparts, outs, bufs)
        torch.cuda.synchronize()
        assert rc == 0
        ref = K.merge_partials(torch.stack(dparts)[:, None])[0]          # [rows, 128]
        for r in range(R):
            assert torch.allclose(outs[r], ref, rtol=1e-5, atol=1e-6), (step, r, float((outs[r] - ref).abs().max()))
            assert torch.equal(outs[r], outs[0]), (step, r)               # every rank merges in the same order
    assert K.lib().fr_device_status() == 0
    # bf16 output: the same sums, rounded once
    last32 = outs[0]
    outs = [torch.zeros(rows, 128, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    assert K.xchg_selftest_step(dparts, outs, bufs) == 0
    torch.cuda.synchronize()
    assert torch.equal(outs[R - 1], last32.bfloat16())


def test_argument_checks():
    from flagrot_releaser_b200 import kernels as K
    L = K.lib()
    import ctypes
    z = torch.zeros(16, device="cuda")
    arr = (ctypes.c_void_p * 9)(*[z.data_ptr()] * 9)
    assert L.fr_xchg_merge(z.data_ptr(), arr, 0, 9, 32, z.data_ptr(), 1, None) == -3      # more than 8 ranks
    assert L.fr_xchg_merge(z.data_ptr(), arr, 2, 2, 32, z.data_ptr(), 1, None) == -3      # rank outside [0, R)
    assert L.fr_xchg_merge(z.data_ptr(), arr, 0, 2, 2000, z.data_ptr(), 1, None) == -3    # more than 1024 rows


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["FR_ROOT"])
from flagrot_releaser_b200 import kernels as K
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
rows = 32
ex = K.ShardExchange(rank, world, rows, dist)
g = torch.Generator().manual_seed(7)
ok = True
for step in range(20):
    parts = [torch.randn(rows, 130, generator=g) for _ in range(world)]
    for p in parts:
        p[:, 128] = torch.randn(rows, generator=g) * 6
        p[:, 129] = torch.rand(rows, generator=g) * 50 + 0.1
    mine = parts[rank].cuda()
    out = torch.zeros(rows, 128, device="cuda")
    ex.merge(mine, out)
    torch.cuda.synchronize()
    ref = K.merge_partials(torch.stack(parts)[:, None])[0]
    ok = ok and torch.allclose(out.cpu(), ref, rtol=1e-5, atol=1e-6)
status = K.lib().fr_device_status()
dist.barrier()
ex.close()
print("RESULT", rank, ok, status, flush=True)
dist.destroy_process_group()
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_two_processes_two_gpus(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    script = tmp_path / "xchg_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, FR_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", WORLD_SIZE=str(world),
               NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o[-2000:]
        assert f"RESULT {r} True 0" in o, o[-2000:]
