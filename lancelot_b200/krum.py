"""Encrypted Krum: the pairwise-distance driver of Lancelot on the B200 path.

Two layers:

* ``GPU_init`` ... ``GPU_krum``: the same functions, argument lists and call sequence as
  ``lancelot-main-GPU/utils/byzantine_fl.py:173-525``, written against
  ``lancelot_b200.pycahel`` so the reference's driver can be pointed at this module unchanged.
* ``EncryptedKrum``: the batched driver.  It keeps context and keys across rounds, encodes and
  encrypts every client ONCE (the reference re-encrypts both clients for every pair,
  byzantine_fl.py:201-212), runs one fused accumulate kernel per pair, then relinearizes,
  rescales and rotate-sums all pairs of a rank as one batch, and shards pairs over ranks.

Per pair the arithmetic is the reference's (byzantine_fl.py:221-273):
    acc = sum over chunks of (ct_j - ct_i)^2            (size 3, scale 2^80, level 1)
    relinearize, rescale to level 2, scale := 2^40
    acc += hoisting(acc, [1..15]); then acc += rot(acc, 2^k) for k = 4 .. log2(slots) - 1
so every slot of the result holds the squared distance.  The reference starts ``acc`` from
square(Enc(0)) instead of zero, which only adds encryption noise; ``EncryptedKrum`` starts
from zero, the compatibility layer keeps the reference's start.
"""
import math
import os
import time

import numpy as np
import torch

from . import pycahel as cahel

# module constants of the reference driver (byzantine_fl.py:23-34)
lazy_relin_flag = 1
Hoisting_flag = 1
Nslot = 32768
log_Nslot = 15


def set_slots(log_slots):
    """The reference hard-codes 32768 slots; other ring degrees need these two changed together."""
    global Nslot, log_Nslot
    log_Nslot = int(log_slots)
    Nslot = 1 << log_Nslot


# ---------------------------------------------------------------------------------------------
# compatibility layer: byzantine_fl.py:173-525 against pycahel
# ---------------------------------------------------------------------------------------------

def GPU_init():
    """byzantine_fl.py:432-463"""
    log_n = log_Nslot + 1
    n = 2 ** log_n
    modulus_chain = [60, 40, 40, 60]
    galois_steps = [i for i in range(1, 16) if i < Nslot]
    galois_steps += [2 ** i for i in range(4, log_n - 1)]
    scale = 2.0 ** 40
    params = cahel.params(cahel.scheme_type.ckks)
    params.set_poly_modulus_degree(n)
    params.set_coeff_modulus(cahel.coeff_modulus_create(n, modulus_chain))
    params.set_special_modulus_size(1)
    params.set_galois_elts(cahel.get_elts_from_steps(galois_steps, n))
    sec = cahel.sec_level_type.tc128 if n >= 8192 else cahel.sec_level_type.none
    context = cahel.context(params, True, sec)
    sk = cahel.secret_key(params)
    sk.gen_secretkey(context)
    pk = cahel.public_key(context)
    sk.gen_publickey(context, pk)
    rlk = cahel.relin_key(context)
    sk.gen_relinkey(context, rlk)
    glk = cahel.galois_key(context)
    sk.create_galois_keys(context, glk)
    encoder = cahel.ckks_encoder(context)
    return context, pk, sk, glk, rlk, encoder, scale


def GPU_compute_pair_distance(msg1, msg2, context, pk, sk, glk, rlk, encoder, scale):
    """byzantine_fl.py:173-323 with lazy relinearization and hoisting (its defaults)"""
    x0 = [0.0] * Nslot
    acc = pk.encrypt_asymmetric(context, encoder.encode(context, x0, scale))
    cahel.square_inplace(context, acc)
    tmp = cahel.ciphertext(context)
    for x1, x2 in zip(msg1, msg2):
        ct1 = pk.encrypt_asymmetric(context, encoder.encode(context, x1, scale))
        ct2 = pk.encrypt_asymmetric(context, encoder.encode(context, x2, scale))
        cahel.sub(context, ct2, ct1, tmp)
        cahel.square_inplace(context, tmp)
        cahel.add_inplace(context, acc, tmp)
    cahel.relinearize_inplace(context, acc, rlk)
    cahel.rescale_to_next_inplace(context, acc)
    acc.set_scale(scale)
    first = [s for s in range(1, 16) if s < Nslot]
    rot = cahel.hoisting(context, acc, glk, first)
    cahel.add_inplace(context, acc, rot)
    tmp_rot = cahel.ciphertext(context)
    for idx in range(4, log_Nslot):
        cahel.rotate_vector(context, acc, int(2 ** idx), glk, tmp_rot)
        cahel.add_inplace(context, acc, tmp_rot)
    return acc


def _pad_and_split(vectors):
    """byzantine_fl.py:478-490: zero-pad to a multiple of the slot count and cut into chunks"""
    weight_len = len(vectors[0])
    whole = weight_len if weight_len % Nslot == 0 else (weight_len // Nslot + 1) * Nslot
    out = []
    for v in vectors:
        p = np.pad(np.asarray(v), (0, whole - weight_len), "constant")
        out.append(np.array_split(p, whole // Nslot))
    return out


def GPU_computing_distance_cipher(context, pk, sk, glk, rlk, encoder, scale, vectors):
    """byzantine_fl.py:466-514; ``vectors`` are the flattened client updates.  Diagonal included, like the reference."""
    vectors_final = _pad_and_split(vectors)
    n = len(vectors_final)
    distance_matrix = [[None] * n for _ in range(n)]
    for i in range(n):
        for j in range(i, n):
            d = GPU_compute_pair_distance(vectors_final[i], vectors_final[j], context, pk, sk, glk, rlk, encoder, scale)
            distance_matrix[i][j] = distance_matrix[j][i] = d
    return distance_matrix, vectors_final


def GPU_decrypt_sort_mask(context, pk, sk, encoder, scale, distance_matrix):
    """byzantine_fl.py:327-369: per client the sum over all pairs, decrypt, slot 0, argsort, one-hot masks"""
    n = len(distance_matrix)
    p_distance = []
    one = pk.encrypt_asymmetric(context, encoder.encode(context, [1.0] * Nslot, scale))
    for i in range(n):
        tmp = pk.encrypt_asymmetric(context, encoder.encode(context, [0.0] * Nslot, scale))
        cahel.mod_switch_to_inplace(context, tmp, 2)
        for j in range(n):
            cahel.add_inplace(context, tmp, distance_matrix[i][j])
        p_distance.append(encoder.decode(context, sk.decrypt(context, tmp))[0])
    order = np.argsort(p_distance)
    zero = pk.encrypt_asymmetric(context, encoder.encode(context, [0.0] * Nslot, scale))
    mask = [[zero for _ in range(n)] for _ in range(n)]
    for i in range(n):
        mask[i][order[i]] = one
    return mask, order[0]


def GPU_mul_mask_weight(context, pk, encoder, scale, rlk, vectors_final, mask, sk):
    """byzantine_fl.py:371-429: sum over clients of weight chunk x mask, size-3 decrypt per chunk"""
    n_clients, n_chunks = len(vectors_final), len(vectors_final[0])
    w_new = []
    tmp = cahel.ciphertext(context)
    pt_zero = encoder.encode(context, [0.0] * Nslot, scale)
    for c in range(n_chunks):
        acc = pk.encrypt_asymmetric(context, pt_zero)
        cahel.square_inplace(context, acc)
        for k in range(n_clients):
            ct2 = pk.encrypt_asymmetric(context, encoder.encode(context, vectors_final[k][c], scale))
            cahel.multiply(context, ct2, mask[0][k], tmp)
            cahel.add_inplace(context, acc, tmp)
        w_new = w_new + encoder.decode(context, sk.decrypt(context, acc))
    return w_new


def GPU_krum(vectors, c=0, args=None):
    """byzantine_fl.py:517-525 on flattened updates; returns the selected (masked) weights"""
    context, pk, sk, glk, rlk, encoder, scale = GPU_init()
    distance_matrix, vectors_final = GPU_computing_distance_cipher(context, pk, sk, glk, rlk, encoder, scale, vectors)
    mask, chosen = GPU_decrypt_sort_mask(context, pk, sk, encoder, scale, distance_matrix)
    return GPU_mul_mask_weight(context, pk, encoder, scale, rlk, vectors_final, mask, sk)


# ---------------------------------------------------------------------------------------------
# batched driver
# ---------------------------------------------------------------------------------------------

def all_pairs(n_clients):
    return [(i, j) for i in range(n_clients) for j in range(i + 1, n_clients)]


def _schedule_for_grid(n_clients, world_size, g):
    size = int(math.ceil(n_clients / g))
    g = int(math.ceil(n_clients / size))
    group = lambda c: c // size
    tiles = {}
    for i, j in all_pairs(n_clients):
        tiles.setdefault((group(i), group(j)), []).append((i, j))
    order = []
    # walk the upper triangle of tiles in a zig-zag so that consecutive tiles share a group
    for a in range(g):
        cols = list(range(a, g))
        if a % 2:
            cols.reverse()
        for b in cols:
            order.extend(tiles.get((a, b), []))
    total = len(order)
    return [order[(total * r) // world_size:(total * (r + 1)) // world_size] for r in range(world_size)]


# Cost of a rank's share in units of one pair's work.  A client the rank must receive costs about three pairs
# (1 GB of ciphertext over NVLink against the accumulate / relinearize / rotate work of one pair) once the
# exchange is no longer hidden behind the encryption, which happens as the ranks' own encryption shrinks:
# the weight grows with the number of ranks (measured: hidden at two ranks, dominant at eight).
def _client_cost(world_size):
    return 3.0 * min(1.0, (world_size - 1) / 4.0)


def _rank_cost(seg, world_size):
    return len(seg) + _client_cost(world_size) * len(clients_of(seg))


def _schedule_by_tiles(n_clients, world_size, g):
    """whole tiles of a g x g grid of client groups handed to ranks, largest first, each to the rank whose cost
    grows least: ranks touch few clients at the price of less even pair counts"""
    size = int(math.ceil(n_clients / g))
    tiles = {}
    for i, j in all_pairs(n_clients):
        tiles.setdefault((i // size, j // size), []).append((i, j))
    segs = [[] for _ in range(world_size)]
    for key in sorted(tiles, key=lambda k: (-len(tiles[k]), k)):
        best = min(range(world_size), key=lambda r: (_rank_cost(segs[r] + tiles[key], world_size), r))
        segs[best].extend(tiles[key])
    return segs


def pair_schedule(n_clients, world_size, kinds=None):
    """Splits the pairs i < j over ``world_size`` ranks so that the busiest rank is as cheap as possible, counting
    its pairs and the distinct clients it touches (it must encrypt or receive each of them).  Candidates: the
    tile-major pair order over a g x g grid of client groups cut into equal contiguous segments ("cuts", the
    default: measured best on eight GPUs), and whole tiles handed out greedily ("tiles": fewer clients per rank,
    less even pair counts; opt in with kinds="cuts,tiles" or LANCELOT_KRUM_SCHEDULE), for every grid size g; one
    rank always gets the plain list.  Every rank must use the same setting."""
    if world_size == 1:
        return [all_pairs(n_clients)]
    best = None
    kinds = (kinds or os.environ.get("LANCELOT_KRUM_SCHEDULE", "cuts")).split(",")
    for g in range(1, n_clients + 1):
        cands = []
        if "cuts" in kinds:
            cands.append((0, _schedule_for_grid(n_clients, world_size, g)))
        if "tiles" in kinds:
            cands.append((1, _schedule_by_tiles(n_clients, world_size, g)))
        for kind, sched in cands:
            key = (max(_rank_cost(seg, world_size) for seg in sched), sum(_rank_cost(seg, world_size) for seg in sched), kind, g)
            if best is None or key < best[0]:
                best = (key, sched)
    return best[1]


def pair_tiles(pairs, width=4):
    """Covers a list of pairs i < j with the tiles lb_krum_accumulate_tile computes in one pass:
    ("tri", clients, []) for all pairs inside a set of 2..width clients, ("rect", rows, cols) for
    1..2 clients against 1..width clients.  Clients are blocked by index in groups of ``width``;
    any pair list is covered, full blocks by the shapes that read least."""
    blocks = {}
    for i, j in pairs:
        blocks.setdefault((i // width, j // width), []).append((i, j))
    tiles = []
    for (ga, gb), ps in sorted(blocks.items()):
        if ga == gb:
            cl = sorted({c for p in ps for c in p})
            if len(ps) == len(cl) * (len(cl) - 1) // 2:
                tiles.append(("tri", cl, []))
                continue
        rows = {}
        for i, j in ps:
            rows.setdefault(i, []).append(j)
        keys = sorted(rows)
        k = 0
        while k < len(keys):
            cols = sorted(rows[keys[k]])
            if k + 1 < len(keys) and sorted(rows[keys[k + 1]]) == cols:
                tiles.append(("rect", [keys[k], keys[k + 1]], cols))
                k += 2
            else:
                tiles.append(("rect", [keys[k]], cols))
                k += 1
    return tiles


def tile_pairs(tile):
    """the pairs of one tile in the order the kernel writes them"""
    kind, rows, cols = tile
    if kind == "tri":
        return [(rows[a], rows[b]) for a in range(len(rows)) for b in range(a + 1, len(rows))]
    return [(i, j) for i in rows for j in cols]


def clients_of(pairs):
    return sorted({c for p in pairs for c in p})


def share_slices(world_size, rank, n_clients, needed_by, produce, alloc, group=None, mark=lambda name: None):
    """Point-to-point exchange of per-client tensors.  Client c is produced by rank c % world_size
    (``produce(c)`` returns its tensor) and sent only to the ranks that list it in ``needed_by[rank]``;
    every rank must call this with the same ``needed_by``.  Clients are handled in slices of world_size
    (one per rank); the transfers of a slice are posted as one batch of isend / irecv and waited for
    after the next slice has been produced, so they overlap with that work.  ``alloc()`` returns an
    empty tensor of a client's shape.  Returns {client: tensor} for the clients this rank needs."""
    import torch.distributed as dist

    out = {}
    pending = None

    def finish(p):
        reqs, keep_alive = p
        for r in reqs:
            r.wait()
        del keep_alive

    for base in range(0, n_clients, world_size):
        c = base + rank
        mine = produce(c) if c < n_clients else None
        mark("encode_encrypt_s")
        ops, hold = [], [mine]
        if mine is not None:
            if c in needed_by[rank]:
                out[c] = mine
            for dst in range(world_size):
                if dst != rank and c in needed_by[dst]:
                    ops.append(dist.P2POp(dist.isend, mine.view(-1), dst, group))
        for src in range(world_size):
            cs = base + src
            if src != rank and cs < n_clients and cs in needed_by[rank]:
                t = alloc()
                out[cs] = t
                ops.append(dist.P2POp(dist.irecv, t.view(-1), src, group))
        reqs = dist.batch_isend_irecv(ops) if ops else []
        if pending is not None:
            finish(pending)
        pending = (reqs, hold)
        mark("ciphertext_exchange_s")
    if pending is not None:
        finish(pending)
    mark("ciphertext_exchange_s")
    return out


_COPY_STREAMS = {}


def _copy_stream(dev):
    """One side stream per device for the whole process: a stream taken fresh from the pool is created
    on first use, and creating a stream while kernels are running can stall for a long time."""
    if dev.index not in _COPY_STREAMS:
        _COPY_STREAMS[dev.index] = torch.cuda.Stream(dev)
    return _COPY_STREAMS[dev.index]


def shared_seed_stream(device, group=None):
    """A seed source (see pycahel.set_seed_source) that gives every rank of the group the same unpredictable stream:
    rank 0 draws 64 bytes from the operating system, broadcasts them, and block k of the stream is
    BLAKE2b(key = those bytes, message = k)."""
    import hashlib

    import torch.distributed as dist

    backend = dist.get_backend(group)
    dev = "cuda:%d" % device if backend == "nccl" else "cpu"
    master = torch.from_numpy(np.frombuffer(os.urandom(64), dtype=np.uint8).copy()).to(dev)
    dist.broadcast(master, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    key = bytes(master.cpu().numpy().tobytes())
    counter = [0]

    def source(count):
        out = bytearray()
        for _ in range(count):
            out += hashlib.blake2b(counter[0].to_bytes(8, "little"), digest_size=64, key=key).digest()
            counter[0] += 1
        return bytes(out)

    return source


class EncryptedKrum:
    """Persistent context + keys, batched encrypt, batched pair scores, plaintext selection.

    log_slots = log2(N/2).  chain {60,40,40 | 60}, scale 2^40 (byzantine_fl.py:432-448)."""

    def __init__(self, log_slots=15, device=None, seed=None, encrypt_batch=384, workspace_bytes=None, rank=0, world_size=1,
                 group=None):
        """rank / world_size / group: the ranks of one job hold the SAME keys.  With ``seed=None`` rank 0 draws a
        64-byte master secret from the operating system and broadcasts it, and every rank expands it with keyed
        BLAKE2b into the same stream of key seeds; the Galois keys (27 switch keys of 12.6 MB at N = 2^16) are
        generated a share per rank and all-gathered instead of being generated by every rank."""
        self.log_slots = log_slots
        self.slots = 1 << log_slots
        self.N = 2 * self.slots
        self.scale = 2.0 ** 40
        self.encrypt_batch = encrypt_batch
        # seed: None = every key and ciphertext seed comes from os.urandom; an integer makes keys and
        # ciphertexts reproducible (tests, benchmarks) and must not be used with real data
        self._rng = np.random.default_rng(seed) if seed is not None else None
        self._test_seed = int(seed) if seed is not None else 0
        steps = [i for i in range(1, 16) if i < self.slots] + [2 ** i for i in range(4, log_slots)]
        self.first_steps = [i for i in range(1, 16) if i < self.slots]
        self.pow_steps = [2 ** i for i in range(4, log_slots)]
        params = cahel.params(cahel.scheme_type.ckks)
        params.set_poly_modulus_degree(self.N)
        params.set_coeff_modulus(cahel.coeff_modulus_create(self.N, [60, 40, 40, 60]))
        params.set_special_modulus_size(1)
        params.set_galois_elts(cahel.get_elts_from_steps(steps, self.N))
        sec = cahel.sec_level_type.tc128 if self.N >= 8192 else cahel.sec_level_type.none
        self.context = cahel.context(params, True, sec, device=device)
        self.lb = self.context.lb
        if workspace_bytes is None:
            # scratch of one fused encode + encrypt call: u, e, two key-level products, the special limbs and
            # the plaintexts of a batch (21 limb-sized rows per ciphertext at this chain); larger batches fill the
            # GPU in whole waves (a 342-ciphertext client in one call is 9 % faster than in batches of 64)
            workspace_bytes = max(5 << 29, int(1.05 * 21 * self.N * 8 * encrypt_batch))
        self.lb.reserve_workspace(workspace_bytes)
        self.steps = steps
        prev = cahel._seed_source
        if self._rng is not None:
            cahel.set_seed_source(lambda k: self._rng.integers(0, 256, 64 * k, dtype=np.uint8))
        elif world_size > 1:
            cahel.set_seed_source(shared_seed_stream(self.lb.device, group))
        try:
            self.sk = cahel.secret_key(params)
            self.sk.gen_secretkey(self.context)
            self.pk = cahel.public_key(self.context)
            self.sk.gen_publickey(self.context, self.pk)
            self.rlk = cahel.relin_key(self.context)
            self.sk.gen_relinkey(self.context, self.rlk)
            self.glk = cahel.galois_key(self.context)
            if world_size > 1:
                self._galois_keys_shared(rank, world_size, group)
            else:
                self.sk.create_galois_keys(self.context, self.glk)
        finally:
            cahel.set_seed_source(prev)
        self.elt_index = {s: self.context.elt_index(e) for s, e in zip(steps, cahel.get_elts_from_steps(steps, self.N))}

    def _galois_keys_shared(self, rank, world_size, group):
        """Galois key i is generated by rank i % world_size; one all-gather hands every rank all of them.  Every rank
        draws every key's seeds from the shared stream, so key i is what a single rank would have generated."""
        import torch.distributed as dist

        ctx, lb = self.context, self.lb
        dnum = ctx.size_Q // ctx.size_P
        n_keys = len(ctx.galois_elts)
        per = (n_keys + world_size - 1) // world_size
        key_shape = (dnum, 2, ctx.size_Q + ctx.size_P, self.N)
        key_words = int(np.prod(key_shape))
        everything = lb.empty(world_size, per, key_words)
        mine = everything[rank]
        all_seeds = [cahel._seeds(2 * dnum) for _ in range(n_keys)]  # every rank draws every key's seeds
        own = list(range(rank, n_keys, world_size))
        if own:
            lb.gen_galois_keys(self.sk.data, own, np.concatenate([all_seeds[i] for i in own]), out=mine[: len(own)])
        dist.all_gather_into_tensor(everything.view(-1), mine.reshape(-1).clone(), group=group)
        self.glk.keys = [everything[i % world_size, i // world_size].view(key_shape) for i in range(n_keys)]

    # -- client side ---------------------------------------------------------------------------
    def n_chunks(self, dim):
        return (dim + self.slots - 1) // self.slots

    def client_seeds(self, client, n_chunks, first_chunk=0):
        """128 seed bytes per ciphertext (ternary u, then the error polynomials).  By default they come from
        the operating system, as the reference draws them for every encryption (cahel-main/include/prng.cuh:12-23):
        whoever can predict them can strip the mask u * pk + e off the ciphertext without the secret key.
        Only an instance built with ``seed=...`` (tests and reproducible benchmarks) derives them from that
        seed, the client index and the chunk range; such an instance must never encrypt real updates."""
        if self._rng is None:
            return np.frombuffer(os.urandom(128 * n_chunks), dtype=np.uint8)
        rng = np.random.default_rng([self._test_seed, int(client), int(first_chunk), 0x4C42])
        return rng.integers(0, 256, 128 * n_chunks, dtype=np.uint8)

    def _as_chunks(self, update):
        """1-D float tensor (any device) -> zero-padded [chunks][slots] on this context's device"""
        dev = "cuda:%d" % self.lb.device
        v = update.to(dev) if isinstance(update, torch.Tensor) else torch.from_numpy(np.asarray(update)).to(dev)
        if v.dtype not in (torch.float32, torch.float64):
            v = v.to(torch.float64)
        dim = v.numel()
        chunks = self.n_chunks(dim)
        pad = chunks * self.slots - dim
        if pad:
            v = torch.cat([v.reshape(-1), torch.zeros(pad, dtype=v.dtype, device=dev)])
        return v.reshape(chunks, self.slots).contiguous()

    def encrypt_chunks(self, values, seeds, out=None):
        """values [k][slots] on the device, seeds 128 bytes per row -> ciphertexts [k][2][3][N] (fused encode + encrypt,
        at most ``encrypt_batch`` per launch group)"""
        k = values.shape[0]
        cts = self.lb.empty(k, 2, 3, self.N) if out is None else out
        for c0 in range(0, k, self.encrypt_batch):
            nb = min(self.encrypt_batch, k - c0)
            self.lb.encode_encrypt(self.pk.data, values[c0:c0 + nb], self.scale, seeds[128 * c0:128 * (c0 + nb)], self.slots, nb,
                                   out=cts[c0:c0 + nb])
        return cts

    def encrypt_client(self, update, client=0, out=None):
        """update: 1-D float32/float64 tensor (CUDA or CPU) -> ciphertexts [chunks][2][3][N]."""
        v = self._as_chunks(update)
        return self.encrypt_chunks(v, self.client_seeds(client, v.shape[0]), out=out)

    def staged(self, updates, clients):
        """Yields (client, update on the device) for the given clients.  Updates that live in host
        memory are copied on a side stream one client ahead of the encryption that consumes them (two
        device buffers), so a pinned host tensor streams in behind the encode + encrypt kernels."""
        if updates.is_cuda:
            for c in clients:
                yield c, updates[c]
            return
        dev = torch.device("cuda", self.lb.device)
        main = torch.cuda.current_stream(dev)
        copy = _copy_stream(dev)
        bufs = [torch.empty(updates.shape[1], dtype=updates.dtype, device=dev) for _ in range(2)]
        ready = [torch.cuda.Event() for _ in range(2)]
        free = [torch.cuda.Event() for _ in range(2)]
        for e in free:
            e.record(main)

        def start(k):
            with torch.cuda.stream(copy):
                copy.wait_event(free[k % 2])
                bufs[k % 2].copy_(updates[clients[k]], non_blocking=True)
                ready[k % 2].record(copy)

        if clients:
            start(0)
        for k, c in enumerate(clients):
            if k + 1 < len(clients):
                start(k + 1)
            main.wait_event(ready[k % 2])
            yield c, bufs[k % 2]
            free[k % 2].record(main)

    def encrypt_slices(self, updates, c_lo, c_hi):
        """Encodes and encrypts chunks [c_lo, c_hi) of EVERY client: updates [n_clients][dim] (CUDA, pinned or pageable
        host) -> ciphertexts [n_clients][c_hi - c_lo][2][3][N].  Several clients' slices share one fused encode + encrypt
        call so that a launch fills the GPU in whole waves even when a rank only holds a few dozen chunks per client;
        rows are copied into a zero-padded staging buffer (on a side stream, one group ahead, when they come from
        host memory)."""
        n_clients, dim = updates.shape
        k = c_hi - c_lo
        e_lo, e_hi = c_lo * self.slots, min(c_hi * self.slots, dim)
        per_call = max(1, self.encrypt_batch // max(k, 1))
        dev = torch.device("cuda", self.lb.device)
        main = torch.cuda.current_stream(dev)
        cts = self.lb.empty(n_clients, k, 2, 3, self.N)
        if k == 0:
            return cts
        groups = [list(range(g, min(g + per_call, n_clients))) for g in range(0, n_clients, per_call)]
        dtype = updates.dtype if updates.dtype in (torch.float32, torch.float64) else torch.float64
        n_buf = 2 if len(groups) > 1 else 1
        bufs = [torch.zeros(per_call, k * self.slots, dtype=dtype, device=dev) for _ in range(n_buf)]
        side = not updates.is_cuda
        copy = _copy_stream(dev) if side else main
        ready = [torch.cuda.Event() for _ in range(n_buf)]
        free = [torch.cuda.Event() for _ in range(n_buf)]
        for e in free:
            e.record(main)

        def start(i):
            b = i % n_buf
            with torch.cuda.stream(copy):
                if side:
                    copy.wait_event(free[b])
                for row, c in enumerate(groups[i]):
                    # one contiguous copy per client: a strided host tensor would go through a pageable temporary
                    bufs[b][row, : e_hi - e_lo].copy_(updates[c, e_lo:e_hi], non_blocking=True)
                if side:
                    ready[b].record(copy)

        start(0)
        for i, grp in enumerate(groups):
            if i + 1 < len(groups) and side:
                start(i + 1)
            b = i % n_buf
            if side:
                main.wait_event(ready[b])
            seeds = np.concatenate([self.client_seeds(c, k, first_chunk=c_lo) for c in grp])
            self.encrypt_chunks(bufs[b][: len(grp)].view(len(grp) * k, self.slots), seeds,
                                out=cts[grp[0]: grp[-1] + 1].view(len(grp) * k, 2, 3, self.N))
            if side:
                free[b].record(main)
            elif i + 1 < len(groups):
                start(i + 1)
        return cts

    # -- server side ---------------------------------------------------------------------------
    def pair_sums(self, cts, pairs, n_slots=None):
        """cts: client -> [chunks][2][3][N] (dict or tensor indexed by client).  Returns acc [n_slots][3][3][N] with
        acc[p] = sum over the chunks of (ct_j - ct_i)^2 for pairs[p] = (i, j); rows past len(pairs) are zero."""
        lb, N = self.lb, self.N
        P = len(pairs)
        n_slots = P if n_slots is None else n_slots
        acc = lb.empty(n_slots, 3, 3, N)
        if n_slots > P:
            acc[P:].zero_()
        if P:
            n_clients = 1 + max(j for _, j in pairs)
            lb.krum_pair_sums(3, cts, n_clients, pairs, acc)  # the tile schedule is chosen inside the library
        return acc

    def finish_scores(self, acc, mark=lambda name: None, stepwise=False):
        """acc [P][3][3][N] (pair sums, scale 2^80, level 1) -> [P][2][2][N]: relinearize, rescale, then the
        rotate-and-sum that leaves the squared distance in every slot (byzantine_fl.py:244-273)"""
        lb, N = self.lb, self.N
        P = acc.shape[0]
        if P == 0:
            return lb.empty(0, 2, 2, N)
        first = [self.elt_index[k] for k in self.first_steps]
        power = [self.elt_index[k] for k in self.pow_steps]
        if stepwise:
            # phases timed apart: the same steps through the single operations
            lb.relinearize_batch(3, acc, self.rlk.data)
            s = lb.rescale_strided(3, acc, P, 2, 3 * 3 * N)  # [P][2][2][N], scale 2^80 / q_2 ~ 2^40
            mark("relin_rescale_s")
            rot = s.clone()
            lb.hoisting_batch(2, rot, first, [self.glk.keys[i] for i in first])
            lb.add(2, s, rot, out=s)
            for e in power:
                rot.copy_(s)
                lb.rotate_batch(2, rot, e, self.glk.keys[e])
                lb.add(2, s, rot, out=s)
            mark("rotate_sum_s")
            return s
        return lb.krum_scores(3, acc, self.rlk.data, first, [self.glk.keys[i] for i in first], power, [self.glk.keys[e] for e in power])

    def pair_scores(self, cts, pairs, mark=lambda name: None, stepwise=False):
        """cts: dict client -> [chunks][2][3][N].  Returns [len(pairs)][2][2][N] level-2 score ciphertexts."""
        if len(pairs) == 0:
            return self.lb.empty(0, 2, 2, self.N)
        acc = self.pair_sums(cts, pairs)
        mark("pair_accumulate_s")
        return self.finish_scores(acc, mark, stepwise)

    def client_sums(self, scores, pairs, n_clients):
        """sum of the score ciphertexts of every pair a client belongs to: [n_clients][2][2][N], one launch"""
        groups = [[p for p, (i, j) in enumerate(pairs) if c in (i, j)] for c in range(n_clients)]
        return self.lb.sum_groups(2, 2, scores.contiguous(), groups)

    def decrypt_slot0(self, ct_level2):
        pt = self.lb.decrypt(2, ct_level2.contiguous(), self.sk.data)
        q2 = self.context.moduli[2]
        # after rescale the true scale is 2^80 / q_2; the reference overwrites it with 2^40 (byzantine_fl.py:246)
        out = self.lb.decode(2, pt, self.scale * self.scale / q2, self.slots)
        return float(out[0].real.item())

    def select(self, sums):
        """decrypt every client's summed distance (slot 0) and return (distances, argsort): one batched decrypt, one
        batched decode and one copy to the host for all clients"""
        n = sums.shape[0]
        pts = self.lb.decrypt_batch(2, sums.contiguous(), self.sk.data, 2, n)
        q2 = self.context.moduli[2]
        # after rescale the true scale is 2^80 / q_2; the reference overwrites it with 2^40 (byzantine_fl.py:246)
        vals = self.lb.decode_batch(2, pts, self.scale * self.scale / q2, self.slots, n)
        d = [float(x) for x in vals[:, 0].real.cpu().tolist()]
        return d, np.argsort(d)

    # -- aggregation phase (byzantine_fl.py:371-429, and the trimmed-mean variant) ---------------------------
    def encrypt_constant(self, value):
        """one ciphertext whose slots all hold ``value`` (the reference's Enc(1) / Enc(0) masks)"""
        dev = "cuda:%d" % self.lb.device
        v = torch.full((1, self.slots), float(value), dtype=torch.float64, device=dev)
        seeds = cahel._seeds(2)
        return self.lb.encode_encrypt(self.pk.data, v, self.scale, seeds, self.slots, 1).reshape(2, 3, self.N)

    def aggregate(self, cts, selected, dim, keep=None):
        """cts: dict client -> [chunks][2][3][N] for ALL clients 0..n-1.  Multiplies every client's ciphertexts
        with its mask ciphertext (Enc(1/k) for the k selected clients, Enc(0) for the rest), adds the products,
        decrypts the size-3 results and decodes them: the plaintext average of the selected updates.
        With one selected client this is GPU_mul_mask_weight; with several it is an encrypted trimmed mean.
        keep: optional dict that receives the mask ciphertexts and the first chunk's size-3 sum (for checks)."""
        lb, N = self.lb, self.N
        n_clients = len(cts)
        chunks = cts[0].shape[0]
        one = self.encrypt_constant(1.0 / len(selected))
        zero = self.encrypt_constant(0.0)
        masks = torch.stack([one if k in set(int(x) for x in selected) else zero for k in range(n_clients)]).contiguous()
        acc = lb.mask_accumulate(3, [cts[k] for k in range(n_clients)], masks, chunks)
        if keep is not None:
            keep["masks"], keep["acc0"] = masks, acc[0].clone()
        pts = lb.decrypt_batch(3, acc, self.sk.data, 3, chunks)
        del acc
        vals = lb.decode_batch(3, pts, self.scale * self.scale, self.slots, chunks)
        return vals.real.reshape(-1)[:dim]

    def aggregate_sharded(self, cts, selected, dim, rank=0, world_size=1, group=None, keep=None):
        """The mask multiplication with the chunk axis sharded over the ranks, as the distance round leaves the
        ciphertexts: cts holds THIS rank's chunk range of every client ([n_clients][k][2][3][N], k = its share of the
        chunks).  Every rank multiplies, decrypts and decodes its chunks; the decoded slices are all-gathered.  Returns
        the averaged update ([dim] float64) on every rank."""
        import torch.distributed as dist

        k = cts[0].shape[0]
        local = self.aggregate(cts, selected, k * self.slots, keep=keep) if k else torch.empty(0, dtype=torch.float64, device="cuda:%d" % self.lb.device)
        if world_size == 1:
            return local[:dim]
        chunks = self.n_chunks(dim)
        most = max(hi - lo for lo, hi in (chunk_range(chunks, r, world_size) for r in range(world_size)))
        send = torch.zeros(most * self.slots, dtype=torch.float64, device=local.device)
        send[: local.numel()] = local
        recv = torch.empty(world_size * most * self.slots, dtype=torch.float64, device=local.device)
        dist.all_gather_into_tensor(recv, send, group=group)
        parts = []
        for r in range(world_size):
            lo, hi = chunk_range(chunks, r, world_size)
            parts.append(recv[r * most * self.slots: r * most * self.slots + (hi - lo) * self.slots])
        return torch.cat(parts)[:dim]

    # -- one round ---------------------------------------------------------------------------------
    def round(self, updates, rank=0, world_size=1, group=None, keep=None, timing=None, exchange="chunks"):
        """updates: [n_clients][dim] tensor (CUDA, pinned or pageable host).  Every rank runs this; rank 0 returns
        (distances, order), the others (None, None).
        exchange: how several ranks share the work.
        "chunks" (default): the pair sum is linear in the chunk axis, so rank r encrypts chunks
        [chunks r / world, chunks (r+1) / world) of EVERY client, forms the partial sums of ALL pairs over its
        chunks, and one reduce-scatter of the partial sums (0.9 GB per rank at 20 clients and N = 2^16, instead
        of the clients' ciphertexts) leaves every rank with the complete sums of its block of pairs; it
        relinearizes, rescales and rotate-sums those, and the scores are all-gathered.  No ciphertext of a
        client ever leaves the GPU that encrypted it.  Residues are below 2^60, so the sum of up to eight
        partial sums fits a signed 64-bit word; it is reduced mod q once afterwards, which equals the
        single-GPU sum word for word.
        "p2p": pairs are sharded instead; client c is encrypted by rank c % world_size and its ciphertexts are
        sent to the ranks whose pairs touch it (batched NCCL isend / irecv overlapped with the next encryption).
        timing: optional dict; when given, the phases are separated by device synchronisations and timed."""
        def mark(name, t=[None]):
            if timing is None:
                return
            torch.cuda.synchronize()
            now = time.perf_counter()
            if t[0] is not None:
                timing[name] = timing.get(name, 0.0) + now - t[0]
            t[0] = now

        mark("start")
        n_clients = updates.shape[0]
        if world_size > 1 and exchange == "p2p":
            return self._round_pair_sharded(updates, rank, world_size, group, keep, mark, stepwise=timing is not None)
        if exchange not in ("chunks", "p2p"):
            raise ValueError("exchange is 'chunks' or 'p2p'")
        import torch.distributed as dist

        pairs = all_pairs(n_clients)
        chunks = self.n_chunks(updates.shape[1])
        c_lo, c_hi = chunk_range(chunks, rank, world_size)
        cts = self.encrypt_slices(updates, c_lo, c_hi)
        mark("encode_encrypt_s")
        block = (len(pairs) + world_size - 1) // world_size
        if world_size > 8:
            raise ValueError("the 64-bit sum of partial pair sums holds for up to eight ranks")
        acc = self.pair_sums(cts, pairs, n_slots=block * world_size)
        mark("pair_accumulate_s")
        if keep is not None:
            keep["cts"], keep["pairs"], keep["partial_sums"] = cts, pairs, acc
        del cts
        if world_size > 1:
            acc = scatter_pair_sums(acc, rank, world_size, group)
            self.lb.reduce_mod(3, acc)
            mark("pair_reduce_scatter_s")
        mine = pairs[rank * block: (rank + 1) * block]
        scores = self.finish_scores(acc[: len(mine)], mark, stepwise=timing is not None)
        del acc
        if keep is not None:
            keep["scores"], keep["my_pairs"] = scores, mine
        # every rank adds the scores of its own pairs into per-client sums (a client's sum is the sum over its pairs, so
        # it splits over the ranks like the pairs do); the partial sums, residues below 2^60 from at most eight
        # ranks, are added as 64-bit words on rank 0 and reduced once: 42 MB per rank instead of a gather of all scores
        sums = self.client_sums(scores, mine, n_clients) if mine else self.lb.empty(n_clients, 2, 2, self.N).zero_()
        if world_size > 1:
            dist.reduce(sums, dst=0 if group is None else dist.get_global_rank(group, 0), op=dist.ReduceOp.SUM, group=group)
            if rank == 0:
                self.lb.reduce_mod(2, sums)
        mark("gather_s")
        if rank != 0:
            return None, None
        out = self.select(sums)
        mark("sum_decrypt_s")
        return out

    def _round_pair_sharded(self, updates, rank, world_size, group, keep, mark, stepwise=False):
        """the "p2p" exchange of round(): pairs sharded over ranks, ciphertexts sent to the ranks that need them"""
        n_clients = updates.shape[0]
        schedule = pair_schedule(n_clients, world_size)
        mine = schedule[rank]
        needed_by = [set(clients_of(seg)) for seg in schedule]
        feed = self.staged(updates, list(range(rank, n_clients, world_size)))
        chunks = self.n_chunks(updates.shape[1])

        def produce(c):
            _, upd = next(feed)
            return self.encrypt_client(upd, client=c)

        cts = share_slices(world_size, rank, n_clients, needed_by, produce, lambda: self.lb.empty(chunks, 2, 3, self.N),
                           group=group, mark=mark)
        scores = self.pair_scores(cts, mine, mark, stepwise=stepwise)
        if keep is not None:
            keep["cts"], keep["scores"], keep["pairs"] = cts, scores, mine
        del cts
        scores, pairs = gather_scores(scores, schedule, rank, world_size, group)
        mark("gather_s")
        if rank != 0:
            return None, None
        sums = self.client_sums(scores, pairs, n_clients)
        out = self.select(sums)
        mark("sum_decrypt_s")
        return out


def chunk_range(n_chunks, rank, world_size):
    """the contiguous chunk range rank ``rank`` of ``world_size`` encrypts and sums"""
    return (n_chunks * rank) // world_size, (n_chunks * (rank + 1)) // world_size


def scatter_pair_sums(partial, rank, world_size, group=None):
    """partial: [world_size * block][...] 64-bit partial sums of every pair over this rank's chunks.  Returns
    [block][...]: the sums over all ranks of block ``rank`` (plain 64-bit addition: the caller reduces mod q).
    NCCL: one reduce-scatter.  gloo (the CPU tests) has no reduce-scatter, so it all-reduces and slices."""
    import torch.distributed as dist

    block = partial.shape[0] // world_size
    if dist.get_backend(group) == "gloo":
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
        return partial[rank * block: (rank + 1) * block].clone()
    out = torch.empty((block,) + tuple(partial.shape[1:]), dtype=partial.dtype, device=partial.device)
    dist.reduce_scatter_tensor(out.view(-1), partial.view(-1), op=dist.ReduceOp.SUM, group=group)
    return out


def gather_scores(local, schedule, rank, world_size, group=None):
    """Gathers the per-rank score ciphertexts on every rank (torch.distributed all_gather, NCCL over
    NVLink on GPUs, gloo in the CPU tests) and returns them with the matching global pair list.
    Segments differ by at most one pair, so shorter ones are padded to the longest."""
    import torch.distributed as dist

    longest = max(len(s) for s in schedule)
    shape = (longest,) + tuple(local.shape[1:])
    send = torch.zeros(shape, dtype=local.dtype, device=local.device)
    send[: local.shape[0]] = local
    recv = [torch.empty_like(send) for _ in range(world_size)]
    dist.all_gather(recv, send, group=group)
    parts, pairs = [], []
    for r in range(world_size):
        k = len(schedule[r])
        parts.append(recv[r][:k])
        pairs.extend(schedule[r])
    return torch.cat(parts, dim=0), pairs


def plaintext_krum(updates):
    """float64 reference of the selection rule as Lancelot applies it (byzantine_fl.py:527-536:
    sum of squared distances to ALL other clients, argmin)."""
    x = updates.to(torch.float64)
    n = x.shape[0]
    d = torch.zeros(n, dtype=torch.float64)
    for i in range(n):
        for j in range(i + 1, n):
            v = float(((x[i] - x[j]) ** 2).sum().item())
            d[i] += v
            d[j] += v
    return d.tolist(), np.argsort(d.numpy())
