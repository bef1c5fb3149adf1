"""The sharded (N > 1) path on CPU: two gloo ranks each own half of the batch, compute their
weight / bias gradients with the oracle, and the all-reduced bucket must equal the full-batch
gradients.  Forward and input-gradient are per-sample, so their shards simply concatenate."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from nectarml_b200.parallel import GradientBucket, shard_range


def test_shard_range_covers_everything():
    for total in (0, 1, 7, 8, 64, 2048):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, world, r) for r in range(world)]
            assert sum(c for _, c in spans) == total
            pos = 0
            for start, count in spans:
                assert start == pos
                pos += count
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import nectar_oracle as orc
        name = "c72"
        case = cases.CONV_CASES[name]
        _, geom, _, _ = case
        B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
        x, w, b, dy = cases.draw_conv(name, case)
        start, count = shard_range(B, world, rank)
        xs, dys = x[start:start + count], dy[start:start + count]
        bucket = GradientBucket([w.shape, (Co,)], "cpu")
        bucket.view(0).copy_(torch.from_numpy(orc.conv2d_backward_weight(dys, xs, w.shape, s, p, d)))
        bucket.view(1).copy_(torch.from_numpy(orc.bias_grad(dys)))
        bucket.all_reduce()
        y_shard = orc.conv2d(xs, w, b, s, p, d)
        ys = [None] * world
        dist.all_gather_object(ys, y_shard)
        if rank == 0:
            full_dw = orc.conv2d_backward_weight(dy, x, w.shape, s, p, d)
            full_db = orc.bias_grad(dy)
            full_y = orc.conv2d(x, w, b, s, p, d)
            ret["dw"] = float(np.abs(bucket.view(0).numpy() - full_dw).max() / np.abs(full_dw).max())
            ret["db"] = float(np.abs(bucket.view(1).numpy() - full_db).max() / np.abs(full_db).max())
            ret["y_equal"] = bool(np.array_equal(np.concatenate(ys, axis=0), full_y))
    finally:
        dist.destroy_process_group()


def test_two_rank_gradient_allreduce_matches_full_batch():
    from oracle import nectar_oracle
    nectar_oracle.build()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret["y_equal"]
        assert ret["dw"] < 2e-6 and ret["db"] < 2e-6


def test_bucket_without_process_group_is_a_noop():
    b = GradientBucket([(3, 4), (5,)], "cpu")
    b.view(0).fill_(1.0)
    assert b.all_reduce() is None
    assert float(b.view(0).sum()) == 12.0 and b.view(1).shape == (5,)


def _store_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nectarml_b200 import train
        store = train.ParamStore("cpu")
        layers = [train._Layer(store, (40, 8, 3, 3), None), train._Layer(store, (16,), (16,)),
                  train._Layer(store, (100, 40), (100,)), train._Layer(store, (7, 5, 1, 1), (7,))]
        store.finalize(n_buckets=3)
        assert store.bucket_bounds[0] == 0 and store.bucket_bounds[-1] == store.n
        assert all(b in [store.offsets[l.ia] for l in layers] + [store.n] for b in store.bucket_bounds[1:])
        # second micro-batch of a step: gradients add to the flat buffer and the buckets leave as they complete
        store.grad.fill_(1.0)
        store.accumulate = True
        store.begin_backward(last_micro_batch=True)
        issued = []
        for l in reversed(layers):  # the backward pass completes the layers last to first

            def run(dw, db, l=l):
                dw.fill_(float(rank + 1))
                if db is not None:
                    db.fill_(10.0 * (rank + 1))
            l.weight_gradient(run)
            issued.append(len(store.pending))
        store.wait_exchange()
        store.accumulate = False
        want_w = sum(1.0 + (r + 1) for r in range(world))
        want_b = sum(1.0 + 10.0 * (r + 1) for r in range(world))
        ok = all(bool((store.g32(l.ia) == want_w).all()) for l in layers)
        ok = ok and all(bool((store.g32(l.ib) == want_b).all()) for l in layers if l.ib is not None)
        if rank == 0:
            ret["ok"] = ok
            ret["issued"] = issued
            ret["buckets"] = len(store.bucket_bounds) - 1
    finally:
        dist.destroy_process_group()


def test_param_store_buckets_leave_as_the_backward_pass_completes_them():
    """Host logic of the training step's gradient exchange on two gloo ranks: flat buffer, bucket cuts at
    layer boundaries, accumulation of a later micro-batch, one all-reduce per bucket issued when the
    bucket's last layer reports in, sums equal over the ranks."""
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_store_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret["ok"]
        assert ret["issued"][-1] == ret["buckets"] and sorted(ret["issued"]) == list(ret["issued"])


def test_only_nets_that_mark_a_frontier_offer_the_split_backward():
    """The data-parallel bench captures the backward pass in two graphs only for nets whose forward() marks
    a frontier; with one micro-batch per GPU (ResNet-50 on 8 GPUs) the other nets take the single graph."""
    from nectarml_b200 import train
    assert train.Pix2PixGenerator.split_backward and not train.ResNet50.split_backward
    assert not train._Net.split_backward


def test_bench_gradient_buckets_are_consecutive_and_front_loaded():
    """The data-parallel sweeps cut their layers into flat gradient buckets in execution order: every layer in
    exactly one bucket, buckets consecutive, each closed bucket at least 8 MB and at least half of what follows
    it, so that the exchange still exposed after the last layer is the smallest one."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    # the Linear sweep under data parallelism: largest gradients first (d = 2048, 2048, 1024, 1024, 512, 512)
    numel = [4 * d * d + 4 * d for d in (2048, 2048, 1024, 1024, 512, 512)]
    groups = bench.bucket_groups(numel, 0.5)
    assert [i for g in groups for i in g] == list(range(len(numel)))
    sizes = [sum(numel[i] for i in g) for g in groups]
    for k, sz in enumerate(sizes[:-1]):
        assert sz * 4 >= (8 << 20) and sz >= 0.5 * sum(sizes[k + 1:])
    assert sizes[-1] == min(sizes) and len(groups) >= 3
    assert bench.bucket_groups([10], 0.5) == [[0]]
    assert bench.bucket_groups([], 0.5) == []
    # tiny layers never close a bucket on their own
    assert bench.bucket_groups([100, 100, 100], 0.5) == [[0, 1, 2]]
