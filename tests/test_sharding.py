"""World-size-2 gloo test (CPU) of the batch-sharding contract: per-sample outputs of the shards
concatenate to the full-batch result, and the all-reduced partial bank gradients equal the
full-batch bank gradient.  The operator itself is played by the CPU oracle (the product has no
CPU path); what is under test is the host-side sharding and reduction logic."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import dk_cases
from deformable_kernels.sharding import allreduce_bank_grad, shard_batch, shard_bounds


def test_shard_bounds_cover_the_batch_once():
    for batch in (1, 2, 7, 128):
        for world in (1, 2, 4, 8):
            cuts = [shard_bounds(batch, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import dk_oracle as O
    O.set_threads(1)
    case = dk_cases.make_case(5, 6, 9, 8, rot_std=1.0, off_std=1.5, seed=50)     # 5 samples over 2 ranks: 3 + 2
    x, o, r, dy = shard_batch([case[k].double() for k in ("input", "offset", "rotation", "grad_output")], rank, world)
    w = case["weight"].double()
    y = O.deform_sample_depthwise_forward(x, o, r, w, **case["args"])
    dx, do, dr, dw = O.deform_sample_depthwise_backward(dy, x, o, r, w, **case["args"])
    allreduce_bank_grad(dw)
    gathered = [None] * world
    dist.all_gather_object(gathered, (y, dx, do, dr))
    if rank == 0:
        q.put((torch.cat([g[0] for g in gathered]), torch.cat([g[1] for g in gathered]),
               torch.cat([g[2] for g in gathered]), torch.cat([g[3] for g in gathered]), dw))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_full_batch():
    from oracle import dk_oracle as O
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as sock:  # a port that is free now, rather than one derived from the pid
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    import queue
    import time
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        result, deadline = None, time.time() + 600   # the children's first `import torch` can take a minute on a cold page cache
        while result is None:
            try:
                result = q.get(timeout=2)
            except queue.Empty:
                dead = [p.exitcode for p in procs if p.exitcode not in (None, 0)]
                assert not dead, "a rank died with exit code %r before the result arrived" % dead
                assert time.time() < deadline, "no result from the ranks within 600 s"
        y, dx, do, dr, dw = result
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
            p.join(timeout=10)
    case = dk_cases.make_case(5, 6, 9, 8, rot_std=1.0, off_std=1.5, seed=50)
    full = {k: case[k].double() for k in ("input", "offset", "rotation", "weight", "grad_output")}
    y0 = O.deform_sample_depthwise_forward(full["input"], full["offset"], full["rotation"], full["weight"], **case["args"])
    g0 = O.deform_sample_depthwise_backward(full["grad_output"], full["input"], full["offset"], full["rotation"],
                                            full["weight"], **case["args"])
    assert torch.equal(y, y0)
    assert torch.equal(dx, g0[0]) and torch.equal(do, g0[1]) and torch.equal(dr, g0[2])
    assert dk_cases.rel_err(dw, g0[3]) < 1e-13
