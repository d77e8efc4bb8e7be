"""The data-parallel exchanges with REAL ranks: one process per GPU over NCCL.  Needs at least two GPUs and is skipped
otherwise; the same host logic runs on one device in test_gpu_level_partition.py (ranks as threads) and on CPU in
test_distributed_cpu.py (gloo)."""
import importlib
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

BASE = dict(grid_resolution=(64,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=3, hash_table_size=1 << 15, growth_factor=1.3819,
            color_hidden_dim=64, color_num_layers=3, lambda_dist=0.01, lambda_depth=0.0, learning_rate=1e-2, beta2=0.99, epsilon=1e-15,
            loss_scale=128.0, density_bias=1.0, bg_color=(1.0, 1.0, 1.0))
RAYS, STEPS = 1 << 12, 6


def _batches(torch, syn):
    scene = syn.SoftSphereScene(); poses = syn.sphere_cameras(20); bg = (1.0, 1.0, 1.0)
    out = []
    for i in range(STEPS):
        o, d = syn.random_training_rays(torch, poses, RAYS, 200, 200, 50.0, seed=900 + i)
        out.append((o, d, syn.ground_truth(torch, scene, o, d, bg)))
    return out


def _rank(rank, world, port, exchange, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        nm = importlib.import_module("3dmaker_b200.nerf"); syn = importlib.import_module("3dmaker_b200.synthetic")
        D = importlib.import_module("3dmaker_b200.distributed")
        eng = nm.InstantNerf(torch, nm.default_options(**dict(BASE, batch_size=(1 << 20) // world, render_batch_size=1 << 18,
                                                              ray_chunk_size=RAYS // world)))
        tr = D.DataParallelTrainer(torch, eng, dist, steps_per_call=1, exchange=exchange)
        for o, d, t in _batches(torch, syn):
            assert tr.train_rays(o, d, t) == RAYS // world
        in_sync = tr.replicas_in_sync()
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, "w_h_%s_%d.npy" % (exchange, rank)), eng.arena_tensor("w_h").float().cpu().numpy())
        np.save(os.path.join(out_dir, "meta_%s_%d.npy" % (exchange, rank)), np.array([int(in_sync), eng.steps.value]))
        tr.close()
        eng.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["peer", "levels", "sharded"])
def test_two_gpus_train_like_one(cuda, nb, tmp_path, exchange):
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    nm = importlib.import_module("3dmaker_b200.nerf"); syn = importlib.import_module("3dmaker_b200.synthetic")
    one = nm.InstantNerf(torch, nm.default_options(**dict(BASE, batch_size=1 << 20, render_batch_size=1 << 18, ray_chunk_size=RAYS)))
    one.set_single_step(True)
    for o, d, t in _batches(torch, syn):
        one.train_rays(o, d, t)
    torch.cuda.synchronize()
    ref = one.arena_tensor("w_h").float().cpu().numpy()
    H = int(one.arena().sparse_count)
    one.close()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank, args=(2, port, exchange, str(tmp_path)), nprocs=2, join=True)
    w0 = np.load(tmp_path / ("w_h_%s_0.npy" % exchange)); w1 = np.load(tmp_path / ("w_h_%s_1.npy" % exchange))
    assert np.array_equal(w0, w1)
    for r in range(2):
        assert list(np.load(tmp_path / ("meta_%s_%d.npy" % (exchange, r)))) == [1, STEPS]
    moved = np.abs(ref[:H] - w0[:H])
    assert np.mean(moved > 2e-3) < 5e-2 and np.mean(moved == 0) > 0.5
    assert np.abs(ref[H:] - w0[H:]).max() <= 5e-2 * np.abs(ref[H:]).max()
