"""Data-parallel training on two GPUs against one GPU: the gradient sums run on a second stream under
back-propagation and into the Adam program, and every Kernel that reads a summed gradient waits for
that sum.  Two ranks with half the batch each must land where one rank with the whole batch lands
(the sums add the ranks' halves in another order: float32 rounding apart).  Needs two GPUs."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["JAXCUDA_REPO"])
from jax_js_b200 import mlp
from jax_js_b200.backend import CudaBackend
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
be = CudaBackend(rank)
uid = [CudaBackend.comm_unique_id() if rank == 0 else None]
dist.broadcast_object_list(uid, src=0)
be.comm_init(rank, world, uid[0])
dims, GB = [784, 1024, 1024, 10], 4096
local = GB // world
rng = np.random.default_rng(5)
x = rng.uniform(0, 1, (GB, dims[0])).astype(np.float32)
y = rng.integers(0, 10, GB).astype(np.int32)
sx, sy = be.put(x[rank * local:(rank + 1) * local]), be.put(y[rank * local:(rank + 1) * local])
out = {}
for mode in ("eager", "graph"):
    tr = mlp.MlpTrainer(be, dims, local, GB, overlap=True)
    losses = []
    for step in range(6):
        if mode == "graph" and step == 1:
            tr.capture(sx, sy, world)
        s = tr.step(sx, sy, world)
        losses.append(float(be.get(s, "float32")[0]))
        be.dec_ref(s)
    out[mode] = (losses, [be.get(p, "float32").copy() for p in tr.params])
    tr.close()
if rank == 0:
    np.savez(os.environ["JAXCUDA_OUT"], eager_loss=out["eager"][0], graph_loss=out["graph"][0],
             **{f"eager_p{i}": p for i, p in enumerate(out["eager"][1])}, **{f"graph_p{i}": p for i, p in enumerate(out["graph"][1])})
dist.barrier()
be.close()
dist.destroy_process_group()
'''


def test_two_ranks_with_overlapped_sums_train_like_one(backend, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from jax_js_b200 import mlp
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script, out = tmp_path / "worker.py", tmp_path / "ranks.npz"
    script.write_text(WORKER)
    env = dict(os.environ, JAXCUDA_REPO=repo, JAXCUDA_OUT=str(out), NCCL_NVLS_ENABLE="0")
    subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                    "--master-port", "29541", str(script)], check=True, env=env, timeout=600)
    got = np.load(out)
    # one rank, whole batch, same seeds
    dims, GB = [784, 1024, 1024, 10], 4096
    rng = np.random.default_rng(5)
    x = rng.uniform(0, 1, (GB, dims[0])).astype(np.float32)
    y = rng.integers(0, 10, GB).astype(np.int32)
    sx, sy = backend.put(x), backend.put(y)
    tr = mlp.MlpTrainer(backend, dims, GB, GB)
    losses = []
    for _ in range(6):
        s = tr.step(sx, sy)
        losses.append(float(backend.get(s, "float32")[0]))
        backend.dec_ref(s)
    params = [backend.get(p, "float32").copy() for p in tr.params]
    tr.close()
    backend.dec_ref(sx)
    backend.dec_ref(sy)
    for mode in ("eager", "graph"):
        np.testing.assert_allclose(got[f"{mode}_loss"], losses, rtol=2e-5, err_msg=mode)
        for i, p in enumerate(params):
            scale = np.abs(p).max()
            assert np.abs(got[f"{mode}_p{i}"] - p).max() <= 2e-3 * scale, (mode, i)   # six Adam steps amplify float32 rounding
    # a sum that a reader overtook would leave a rank with half the gradient: far outside these bounds
