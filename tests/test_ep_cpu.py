"""Expert-parallel host logic on CPU: world_size-2 (and 4) gloo ranks run the dispatch ->
local experts -> combine exchange with the row layout of the C ABI (moe_ep_layout, the same
arithmetic a GPU forward runs on the host) and must reproduce the single-device oracle on the
concatenated batch.  No GPU, no NCCL."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _p2p_exchange(recv, send, rank, world):
    """Grouped send/recv between every pair of ranks (what ncclGroupStart..ncclSend/ncclRecv..
    ncclGroupEnd does on the GPU path); a rank's own chunk is a local copy; empty chunks are
    skipped on both sides, which both know from the gathered counts."""
    reqs = []
    for r in range(world):
        if r == rank:
            recv[r].copy_(send[r])
            continue
        if send[r].numel():
            reqs.append(dist.isend(send[r], dst=r))
        if recv[r].numel():
            reqs.append(dist.irecv(recv[r], src=r))
    for q_ in reqs:
        q_.wait()


def _rank_main(rank, world, port, E, k, T, D, H, O, tile_m, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mixtureofexperts_b200 import parallel
        from oracle import moe_oracle as orc

        # every rank draws the whole problem; it owns tokens [rank*T, (rank+1)*T) and E/world experts
        x_all, w = orc.make_layer_inputs(99, T * world, D, H, O, E, init="normal", std=0.25)
        cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                            gate_type=orc.TopKGating(k), balance_alpha=0.01, z_loss_weight=0.001)
        x = x_all[rank * T:(rank + 1) * T]
        idx, gates, probs, logits = orc.router_forward(cfg, w, x)

        uid = parallel.broadcast_unique_id(dist, rank, None, make_id=lambda: bytes(range(128)))
        assert uid == bytes(range(128))
        mine = parallel.expert_partition(E, world, rank)
        per = len(mine)

        counts = np.bincount(idx.ravel() - 1, minlength=E).astype(np.int32)
        cnt = parallel.all_gather_counts(dist, counts, rank, timeout_s=60.0)
        send_off, recv_off, local_off, tile_prefix, rows = parallel.exchange_layout(cnt, rank, tile_m)
        assert rows == cnt[:, mine.start:mine.stop].sum()
        assert tile_prefix[-1] == sum((cnt[:, e].sum() + tile_m - 1) // tile_m for e in mine)

        # permute: pairs in (expert, token, slot) order, the order the permute kernel produces
        tok = np.repeat(np.arange(T), k)
        flat_e = idx.ravel() - 1
        order = np.argsort(flat_e, kind="stable")
        pair_pos = np.empty(T * k, dtype=np.int64)
        pair_pos[order] = np.arange(T * k)
        xs = x[tok[order]]
        assert all(np.all(flat_e[order][send_off[e]:send_off[e + 1]] == e) for e in range(E))

        # dispatch: one message per peer holding its experts' rows in expert order
        send = [torch.from_numpy(np.ascontiguousarray(xs[send_off[r * per]:send_off[(r + 1) * per]])) for r in range(world)]
        recv = [torch.zeros((int(cnt[r, mine.start:mine.stop].sum()), D), dtype=torch.float32) for r in range(world)]
        _p2p_exchange(recv, send, rank, world)
        xr = np.zeros((rows, D), dtype=np.float32)
        for r in range(world):
            o = 0
            for el in range(per):
                n = int(cnt[r, mine.start + el])
                xr[recv_off[el, r]:recv_off[el, r] + n] = recv[r].numpy()[o:o + n]
                o += n
        # local experts on the received rows
        yr = np.zeros((rows, O), dtype=np.float32)
        for el in range(per):
            a, b = local_off[el], local_off[el + 1]
            if b > a:
                yr[a:b] = orc.gated_expert_forward(w.experts[mine.start + el], xr[a:b], orc.silu)
        # combine: rows back to their owners, into the send layout
        back = []
        for r in range(world):
            parts = [yr[recv_off[el, r]:recv_off[el, r] + int(cnt[r, mine.start + el])] for el in range(per)]
            back.append(torch.from_numpy(np.ascontiguousarray(np.concatenate(parts)) if parts else np.zeros((0, O), np.float32)))
        got = [torch.zeros((int(send_off[(r + 1) * per] - send_off[r * per]), O), dtype=torch.float32) for r in range(world)]
        _p2p_exchange(got, back, rank, world)
        y_back = np.zeros((T * k, O), dtype=np.float32)
        for r in range(world):
            y_back[send_off[r * per]:send_off[(r + 1) * per]] = got[r].numpy()
        out = np.zeros((T, O), dtype=np.float32)
        for t in range(T):
            slots = sorted(range(k), key=lambda s: idx[t, s])
            for s in slots:
                out[t] += gates[t, s] * y_back[pair_pos[t * k + s]]
        # loss from all-reduced sums
        sums = np.concatenate([counts.astype(np.float64), probs.sum(axis=0, dtype=np.float64),
                               [float((orc.logsumexp_dim1(logits) ** 2).sum()), float(T)]])
        ts = torch.from_numpy(sums)
        dist.all_reduce(ts)
        s = ts.numpy()
        Tg = s[-1]
        loss = 0.01 * E * np.sum((s[:E] / (k * Tg)) * (s[E:2 * E] / Tg)) + 0.001 * s[2 * E] / Tg

        ref_out, ref_loss, _ = orc.moe_layer_forward(cfg, w, x_all, training=True)
        err = np.abs(out - ref_out[rank * T:(rank + 1) * T]).max() / np.abs(ref_out).max()
        q.put((rank, float(err), float(abs(loss - ref_loss) / abs(ref_loss))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,E,k,T", [(2, 8, 2, 37), (4, 8, 2, 16), (2, 4, 1, 5)])
def test_expert_parallel_exchange_matches_single_device_oracle(lib_built, world, E, k, T):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 500) + world
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, E, k, T, 32, 48, 24, 4, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=5) for _ in range(world))
    assert [r[0] for r in results] == list(range(world))
    for _, err, lerr in results:
        assert err < 1e-5 and lerr < 1e-5


def test_layout_of_a_hand_checked_case(lib_built):
    from mixtureofexperts_b200 import parallel

    # 2 ranks, 4 experts (2 per rank); counts[r][e]
    cnt = np.array([[3, 0, 2, 1], [1, 4, 0, 2]], dtype=np.int32)
    so, ro, lo, tp, rows = parallel.exchange_layout(cnt, 1, 2)
    assert so.tolist() == [0, 1, 5, 5, 7]
    # rank 1 owns experts 2,3: expert 2 gets 2 rows from rank 0 and 0 from itself, expert 3 gets 1 + 2
    assert ro.tolist() == [[0, 2], [2, 3]] and lo.tolist() == [0, 2, 5] and rows == 5
    assert tp.tolist() == [0, 1, 3]
    with pytest.raises(Exception):
        parallel.exchange_layout(np.zeros((3, 4), dtype=np.int32), 0, 2)  # 4 experts over 3 ranks


def test_layout_rejects_count_vectors_that_no_router_produced(lib_built):
    """moe_ep_layout is what every rank runs on the gathered counts: a negative count, or more rows
    than an int32 row index can address, must be refused (the forward then fails on every rank
    alike, because all ranks look at the same table)."""
    from mixtureofexperts_b200 import _lib, parallel

    bad = np.array([[3, 0, 2, 1], [1, -4, 0, 2]], dtype=np.int32)
    with pytest.raises(_lib.MoEError) as ei:
        parallel.exchange_layout(bad, 0, 2)
    assert ei.value.code == _lib.ERR_INVALID
    huge = np.full((2, 4), 2**30, dtype=np.int32)
    with pytest.raises(_lib.MoEError) as ei:
        parallel.exchange_layout(huge, 1, 128)
    assert ei.value.code == _lib.ERR_UNSUPPORTED


def _absent_rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    import time

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        from mixtureofexperts_b200 import _lib, parallel

        counts = np.arange(8, dtype=np.int32) + rank
        cnt = parallel.all_gather_counts(dist, counts, rank, timeout_s=30.0)       # everybody posts: fine
        assert cnt.shape == (world, 8) and np.array_equal(cnt[rank], counts)
        if rank == 0:
            t0 = time.perf_counter()
            try:
                parallel.all_gather_counts(dist, counts, rank, timeout_s=1.5)       # rank 1 stays away
                q.put((rank, "no error", 0.0))
            except _lib.MoEError as exc:
                q.put((rank, exc.code, time.perf_counter() - t0))
        else:
            time.sleep(4.0)                                                          # never posts its counts
            q.put((rank, "absent", 0.0))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001  (the group is broken on purpose)
            pass


def test_a_rank_that_never_posts_its_counts_costs_a_timeout_not_a_hang(lib_built):
    from mixtureofexperts_b200 import _lib

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 500) + 11
    procs = [ctx.Process(target=_absent_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode is not None, "a rank is still waiting"
    results = dict((r[0], r[1:]) for r in (q.get(timeout=5) for _ in range(2)))
    code, waited = results[0]
    assert code == _lib.ERR_TIMEOUT and waited < 30.0
    assert results[1][0] == "absent"


def _disagree_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mixtureofexperts_b200 import _lib, parallel

        counts = np.array([2, 1, 0, 3], dtype=np.int32)
        # rank 1's transport hands back a table whose own row is not what it posted
        class Tampering:
            def get_world_size(self):
                return dist.get_world_size()

            def all_gather(self, out, t, async_op=False):
                w = dist.all_gather(out, t, async_op=async_op)
                if rank == 1:
                    if w is not None:
                        w.wait()
                    out[1][0] += 5
                return w

        try:
            parallel.all_gather_counts(Tampering(), counts, rank, timeout_s=30.0)
            q.put((rank, "ok"))
        except _lib.MoEError as exc:
            q.put((rank, exc.code))
    finally:
        dist.destroy_process_group()


def test_count_vectors_that_disagree_with_what_was_posted_are_refused(lib_built):
    from mixtureofexperts_b200 import _lib

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 500) + 17
    procs = [ctx.Process(target=_disagree_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=5) for _ in range(2))
    assert results[0] == "ok" and results[1] == _lib.ERR_NCCL


def test_numa_binding_reads_sysfs_and_leaves_unknown_topologies_alone(tmp_path):
    """bind_to_gpu_numa_node: the node's CPU list (restricted to what the process may use) becomes
    the affinity mask; an unknown node, a missing device or a foreign CPU list changes nothing."""
    import os

    from mixtureofexperts_b200 import parallel

    before = os.sched_getaffinity(0)
    try:
        dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
        dev.mkdir(parents=True)
        node = tmp_path / "devices/system/node/node1"
        node.mkdir(parents=True)
        mine = sorted(before)
        keep = mine[: max(1, len(mine) // 2)]
        (dev / "numa_node").write_text("1\n")
        (node / "cpulist").write_text(",".join(str(c) for c in keep) + ",100000-100003\n")
        got = parallel.bind_to_gpu_numa_node("00000000:1B:00.0", sysfs=str(tmp_path))
        assert got == {"node": 1, "cpus": len(keep)}
        assert os.sched_getaffinity(0) == set(keep)
        os.sched_setaffinity(0, before)
        (dev / "numa_node").write_text("-1\n")
        assert parallel.bind_to_gpu_numa_node("0000:1b:00.0", sysfs=str(tmp_path))["node"] == -1
        assert parallel.bind_to_gpu_numa_node("0000:99:00.0", sysfs=str(tmp_path))["node"] == -1
        (dev / "numa_node").write_text("1\n")
        (node / "cpulist").write_text("100000-100003\n")
        assert parallel.bind_to_gpu_numa_node("1b:00.0", sysfs=str(tmp_path))["node"] == -1
        assert os.sched_getaffinity(0) == before
    finally:
        os.sched_setaffinity(0, before)
