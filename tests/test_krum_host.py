"""Host-side logic of the Krum driver: pair scheduling and the world_size-2 gather (gloo, CPU)."""
import math
import os

import numpy as np
import pytest
import torch


def test_pair_schedule_covers_every_pair_once_and_balances():
    from lancelot_b200.krum import all_pairs, clients_of, pair_schedule

    for n in (2, 4, 10, 20, 33):
        for world in (1, 2, 4, 8):
            sched = pair_schedule(n, world)
            assert len(sched) == world
            flat = [p for s in sched for p in s]
            assert sorted(flat) == all_pairs(n)
            sizes = [len(s) for s in sched]
            # pair counts stay close to even: nobody carries more than a third above the mean (plus one)
            assert max(sizes) <= 1 + math.ceil(len(flat) / world * 4 / 3)
    # two ranks: the exchange hides behind the encryption, so the split is the even one
    sizes = [len(s) for s in pair_schedule(20, 2)]
    assert max(sizes) - min(sizes) <= 1
    # eight ranks: a rank touches at most 13 of the 20 clients with equal cuts, 10 when whole tiles may be handed out
    sched = pair_schedule(20, 8)
    assert max(len(clients_of(s)) for s in sched) <= 13 and max(len(s) for s in sched) - min(len(s) for s in sched) <= 1
    sched = pair_schedule(20, 8, kinds="cuts,tiles")
    assert sorted(p for s in sched for p in s) == all_pairs(20)
    assert max(len(clients_of(s)) for s in sched) <= 10 and max(len(s) for s in sched) <= 25


def test_pair_tiles_cover_every_pair_once_with_valid_shapes():
    from lancelot_b200.krum import all_pairs, pair_schedule, pair_tiles, tile_pairs

    reads = 0
    for n in (2, 3, 5, 10, 20, 33):
        for world in (1, 2, 3, 8):
            for part in pair_schedule(n, world):
                tiles = pair_tiles(part)
                covered = [p for t in tiles for p in tile_pairs(t)]
                assert sorted(covered) == sorted(part) and len(covered) == len(set(covered))
                for kind, rows, cols in tiles:
                    if kind == "tri":
                        assert 2 <= len(rows) <= 4 and not cols
                    else:
                        assert 1 <= len(rows) <= 2 and 1 <= len(cols) <= 4
                        assert all(i < j for i in rows for j in cols)
                if n == 20 and world == 1:
                    reads = sum(len(r) + len(c) for _, r, c in tiles)
    # 20 clients on one rank: 140 client reads instead of 2 x 190
    assert reads == 140 and len(all_pairs(20)) == 190


def test_plaintext_krum_rule():
    from lancelot_b200.krum import plaintext_krum

    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 50, generator=g) * 0.01
    x[4] += 1.0  # an outlier has the largest summed distance
    d, order = plaintext_krum(x)
    assert order[-1] == 4 and len(d) == 6
    i, j = 1, 3
    xd = x.double()
    assert abs(sum(float(((xd[i] - xd[k]) ** 2).sum()) for k in range(6) if k != i) - d[i]) < 1e-9


def _gather_worker(rank, world, port, ret):
    import torch.distributed as dist

    from lancelot_b200.krum import gather_scores, pair_schedule

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n_clients = 5  # 10 pairs over 2 ranks; with 3 ranks segments would be uneven
        sched = pair_schedule(n_clients, world)
        mine = sched[rank]
        # a fake "score ciphertext" whose words encode the pair it belongs to
        local = torch.stack([torch.full((2, 2, 8), 100 * i + j, dtype=torch.int64) for i, j in mine])
        scores, pairs = gather_scores(local, sched, rank, world)
        ok = len(pairs) == 10 and all(int(scores[k, 0, 0, 0]) == 100 * i + j for k, (i, j) in enumerate(pairs))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_gather_scores_world_size_n_gloo(world):
    import torch.multiprocessing as mp

    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 500) + world
    mp.spawn(_gather_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def _p2p_worker(rank, world, port, n_clients, out):
    import torch.distributed as dist

    from lancelot_b200.krum import clients_of, pair_schedule, share_slices

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        schedule = pair_schedule(n_clients, world)
        needed_by = [set(clients_of(seg)) for seg in schedule]
        produced = []

        def produce(c):
            produced.append(c)
            return torch.full((6,), float(c) + 0.5)

        got = share_slices(world, rank, n_clients, needed_by, produce, lambda: torch.empty(6))
        ok = sorted(got) == sorted(needed_by[rank]) and all(float(t[0]) == c + 0.5 and float(t[-1]) == c + 0.5 for c, t in got.items())
        ok = ok and produced == list(range(rank, n_clients, world))
        out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_clients", [(2, 5), (3, 7), (4, 20)])
def test_point_to_point_ciphertext_exchange_gloo(world, n_clients):
    """every rank ends up with exactly the clients its pairs touch, each produced once by its owner"""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29610 + world
    procs = [ctx.Process(target=_p2p_worker, args=(r, world, port, n_clients, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, True) for r in range(world)]


def _chunk_worker(rank, world, port, out):
    import torch.distributed as dist

    from lancelot_b200.krum import all_pairs, chunk_range, scatter_pair_sums
    from oracle import binding

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        logn, L, n_clients, chunks = 8, 3, 5, 7
        n = 1 << logn
        mods = binding.coeff_modulus_create(n, [60, 40, 40, 60])
        o = binding.Oracle(logn, mods, 1)
        rng = np.random.default_rng(42)  # every rank draws the same "ciphertexts"
        cts = np.stack([np.stack([rng.integers(0, mods[r], n, dtype=np.uint64) for r in range(L)] * 2).reshape(2, L, n)
                        for _ in range(n_clients * chunks)]).reshape(n_clients, chunks, 2, L, n)
        cts[0, 0] = 0
        for r in range(L):
            cts[1, 0][:, r, :] = mods[r] - 1  # largest residues: the 64-bit sum of partial sums must not wrap
        pairs = all_pairs(n_clients)

        def pair_sum(i, j, lo, hi):
            acc = np.zeros((3, L, n), dtype=np.uint64)
            for c in range(lo, hi):
                acc = o.poly_op("add", L, acc, o.square(L, o.poly_op("sub", L, cts[j, c], cts[i, c]).reshape(2, L, n)))
            return acc

        lo, hi = chunk_range(chunks, rank, world)
        block = (len(pairs) + world - 1) // world
        partial = np.zeros((block * world, 3, L, n), dtype=np.uint64)
        for p, (i, j) in enumerate(pairs):
            partial[p] = pair_sum(i, j, lo, hi)
        mine = scatter_pair_sums(torch.from_numpy(partial.view(np.int64)), rank, world).numpy().view(np.uint64)
        q = np.array(mods[:L], dtype=np.uint64).reshape(1, 1, L, 1)
        mine = mine % q
        ok = True
        for k, (i, j) in enumerate(pairs[rank * block:(rank + 1) * block]):
            ok = ok and np.array_equal(mine[k], pair_sum(i, j, 0, chunks))
        ok = ok and not mine[len(pairs[rank * block:(rank + 1) * block]):].any()
        out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_chunk_sharded_pair_sums_equal_single_rank_sums_gloo(world):
    """ranks sum the pairs over their own chunk ranges; the scattered 64-bit sums, reduced mod q once, equal the
    sums one rank forms over all chunks, word for word"""
    import torch.multiprocessing as mp

    from lancelot_b200.krum import chunk_range

    assert [chunk_range(342, r, 8) for r in (0, 7)] == [(0, 42), (299, 342)]
    assert sum(hi - lo for lo, hi in (chunk_range(7, r, 4) for r in range(4))) == 7
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29710 + world
    procs = [ctx.Process(target=_chunk_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, True) for r in range(world)]


def _seed_stream_worker(rank, world, port, out):
    import hashlib

    import torch.distributed as dist

    from lancelot_b200.krum import shared_seed_stream

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        src = shared_seed_stream(0)
        a, b = src(3), src(2)
        out.put((rank, len(a), len(b), hashlib.sha256(a + b).hexdigest(), a[:64] != a[64:128] and a[:64] != b[:64]))
    finally:
        dist.destroy_process_group()


def test_ranks_expand_one_broadcast_secret_into_the_same_key_seeds_gloo():
    """several ranks must hold the same keys: rank 0's 64 random bytes reach every rank and give the same stream"""
    import torch.multiprocessing as mp

    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_seed_stream_worker, args=(r, world, 29731, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert [r[0] for r in res] == list(range(world))
    assert all(r[1] == 192 and r[2] == 128 and r[4] for r in res)
    assert len({r[3] for r in res}) == 1


def test_rotation_steps_decompose_like_the_reference():
    """non-adjacent form, least significant term first: the order the reference key-switches a rotation step that
    has no key of its own (cahel-main/include/util/numth.h:18-35, src/evaluate.cu:2396-2407); the reference-made
    fixture entry "rotate_naf" pins that the order matters bit for bit"""
    from lancelot_b200.pycahel import _naf

    assert _naf(5) == [1, 4]
    assert _naf(6) == [-2, 8]
    assert _naf(3) == [-1, 4]
    assert _naf(-3) == [1, -4]
    assert _naf(16) == [16]
    for v in range(-70, 71):
        parts = _naf(v)
        assert sum(parts) == v
        mags = [abs(p) for p in parts]
        assert mags == sorted(mags) and all(m & (m - 1) == 0 for m in mags)
        assert all(b >= 4 * a for a, b in zip(mags, mags[1:]))  # no two adjacent powers
