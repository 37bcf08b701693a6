"""Benchmark workloads beyond the plain NTT sweep: the encrypted-Krum distance round
(BASELINE configs 3 and 4) and the multiply + relinearize + rescale chain at N = 2^16, L = 24.

Each class follows the small protocol bench.py drives: setup_gpu / step_gpu / step_e2e /
check_gpu / cpu_sample, plus the bookkeeping the JSON line needs.  Inputs are seeded synthetic
tensors with the shapes and value distributions BASELINE.json names (no dataset exists here)."""
import ctypes as C
import os
import time

import numpy as np


def _launches():
    from ._lib import lib

    lib.lb_launch_count.restype = C.c_ulonglong
    return int(lib.lb_launch_count())


class KrumWorkload:
    """Encrypted Krum, distance phase: context + keys, encode + encrypt of every client this rank
    needs, fused pair accumulation, batched relinearize / rescale / rotate-and-sum, gather of the
    score ciphertexts, per-client sums, decryption, argsort.  Default is BASELINE configs[4]
    (ResNet-18 scale, 20 clients, N = 2^16); --batch 10 selects configs[3] (MNIST-CNN scale, N = 2^15)."""
    name = "krum"
    metric = "encrypted_krum_round_s"
    unit = "s"
    higher_is_better = False
    dtype = "u64"
    scaling = "strong"

    def __init__(self, batch=20):
        self.n_clients = int(batch)
        if self.n_clients == 10:
            self.dim, self.log_slots, self.n_byz, self.tag = 1663370, 14, 2, "C4"
        else:
            self.dim, self.log_slots, self.n_byz, self.tag = 11173962, 15, 4, "C5"
        self.slots = 1 << self.log_slots
        self.chunks = (self.dim + self.slots - 1) // self.slots
        self.launches_per_step = 0
        self.breakdown = {}
        self.profile_phases = False
        # how ciphertexts reach the ranks that need them when several GPUs share a round (EncryptedKrum.round)
        self.exchange = os.environ.get("LANCELOT_KRUM_EXCHANGE", "p2p")

    def config(self):
        return {"workload": "%s encrypted Krum distance round: %d clients x %d float32, N=2^%d, %d ciphertexts per client, "
                            "%d pairs, chain {60,40,40|60}, scale 2^40" % (self.tag, self.n_clients, self.dim, self.log_slots + 1,
                                                                          self.chunks, self.n_clients * (self.n_clients - 1) // 2),
                "l2": "inputs (%.1f GiB of ciphertext) exceed the 126 MB L2" % (self.n_clients * self.chunks * 6 * (2 * self.slots) * 8 / 2 ** 30),
                "includes": "context + key generation, encode, encrypt, pair distances, score gather, decrypt, argsort",
                "excludes": "mask multiplication phase (GPU_mul_mask_weight)"}

    # -- data ------------------------------------------------------------------------------------
    def make_updates(self, device):
        import torch
        g = torch.Generator(device=device)
        g.manual_seed(20240)
        x = torch.randn(self.n_clients, self.dim, generator=g, device=device, dtype=torch.float32) * 1e-2
        if self.tag == "C4":
            x[: self.n_byz] = torch.randn(self.n_byz, self.dim, generator=g, device=device, dtype=torch.float32)
        else:
            x[: self.n_byz] += (torch.rand(self.n_byz, self.dim, generator=g, device=device, dtype=torch.float32) * 10 - 5)
        return x

    def setup_gpu(self, device):
        import torch
        import torch.distributed as dist
        self.torch = torch
        self.device = device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        dev = "cuda:%d" % device
        self.updates = self.make_updates(dev)
        self.host = torch.empty(self.updates.shape, dtype=torch.float32).pin_memory()
        self.host.copy_(self.updates)
        self.result = None
        # float64 plaintext Krum on the device, for the parity check
        n = self.n_clients
        d = torch.zeros(n, dtype=torch.float64, device=dev)
        for i in range(n):
            for j in range(i + 1, n):
                v = ((self.updates[i].double() - self.updates[j].double()) ** 2).sum()
                d[i] += v
                d[j] += v
        self.want = d.cpu().numpy()

    def _round(self, updates):
        from . import krum
        t0 = time.perf_counter()
        l0 = _launches()
        ek = krum.EncryptedKrum(log_slots=self.log_slots, device=self.device, seed=1)
        self.torch.cuda.synchronize()
        t1 = time.perf_counter()
        timing = {} if self.profile_phases else None
        d, order = ek.round(updates, rank=self.rank, world_size=self.world, timing=timing, exchange=self.exchange)
        self.torch.cuda.synchronize()
        t2 = time.perf_counter()
        self.launches_per_step = _launches() - l0
        if timing:
            self.breakdown = {"init_s": t1 - t0, "round_s": t2 - t1}
            self.breakdown.update({k: v for k, v in timing.items() if k != "start"})
        self.result = (d, order)
        del ek
        if timing:
            self.torch.cuda.synchronize()
            self.breakdown["teardown_s"] = time.perf_counter() - t2

    def step_gpu(self):
        self._round(self.updates)

    def step_e2e(self):
        # the round takes the pinned host tensor itself: it copies one client ahead of the encryption
        self._round(self.host)
        out_bytes = 8 * self.n_clients * 2
        return self.host.numel() * 4, out_bytes

    def check_gpu(self):
        if self.rank != 0 or self.result is None or self.result[0] is None:
            return True
        d, order = self.result
        rel = float(np.max(np.abs(np.array(d) - self.want) / self.want))
        self.rel_err = rel
        return bool(rel < 1e-6 and list(order) == list(np.argsort(self.want)))

    def units_per_step(self):
        return 1.0

    def algorithmic_bytes_per_step(self):
        pairs = self.n_clients * (self.n_clients - 1) // 2
        return pairs * 2 * self.chunks * 6 * (2 * self.slots) * 8

    # -- dominant kernel -------------------------------------------------------------------------------
    def time_dominant_kernel(self, timed):
        """The forward transform takes the largest share of a round (see the launch shares under profiles/):
        timed alone on 64 key-level polynomials of this chain ({60,40,40|60}: 256 limbs, 128 MiB > L2).
        The pair accumulation tile (2 x 4 clients, the round's second kernel) is timed too and reported
        as ``roofline_pair_kernel``."""
        from . import krum
        torch = self.torch
        ek = krum.EncryptedKrum(log_slots=self.log_slots, device=self.device, seed=1)
        lb, N = ek.lb, ek.N
        polys = 64
        g = torch.Generator(device="cuda:%d" % self.device)
        g.manual_seed(7)
        data = torch.randint(0, 1 << 39, (polys, 4, N), dtype=torch.int64, device="cuda:%d" % self.device, generator=g)
        fn = lambda: lb.ntt_forward(data, polys, 3, 1)
        for _ in range(3):
            fn()
        ms, _ = timed(fn, 10)
        self._kernel_bytes = 16 * N * 4 * polys
        per_limb = (N // 2) * (self.log_slots + 1)
        # half of the limbs take the integer butterfly (60-bit primes), half the FP64-assisted lazy one (40-bit)
        roofs = [lb.butterfly_rate(v) / per_limb * 16 * N / 1e9 for v in (0, 3)]
        self.int_roof_gbs = 2.0 / (1.0 / roofs[0] + 1.0 / roofs[1])
        del data
        # pair tile: two clients against four
        cl = [ek.encrypt_client(self.updates[i], client=i) for i in range(6)]
        outs = [lb.empty(3, 3, N) for _ in range(8)]
        tile = lambda: lb.krum_accumulate_tile(3, cl[:2], cl[2:], outs)
        for _ in range(2):
            tile()
        tms, _ = timed(tile, 5)
        tile_bytes = 6 * cl[0].numel() * 8 + 8 * outs[0].numel() * 8
        self.pair_kernel = {"kernel": "krum_tile_kernel<2,4>", "bound": "hbm", "achieved": tile_bytes / (tms / 5 * 1e-3) / 1e9, "unit": "GB/s",
                            "bytes_per_launch": tile_bytes, "pairs_per_launch": 8}
        del cl, outs
        return ms / 10, "ntt_fwd_fixed_kernel<3> (plain input)"

    def roofline_kernel_bytes(self):
        return self._kernel_bytes

    @property
    def ncu_traffic_bytes(self):
        # one captured launch of this kernel moved 404.1 MB of DRAM traffic for 402.7 MB of algorithmic
        # bytes (16 polynomials x 24 limbs); traffic grows with the limb count, so the ratio carries over
        return int(self._kernel_bytes * 404.1 / 402.7)

    # -- CPU baseline -----------------------------------------------------------------------------------
    def cpu_sample(self, threads):
        """Oracle timed on one ciphertext's encode + encrypt, one chunk of one pair, and one pair's
        relinearize / rescale / rotate-and-sum; the round time is extrapolated from the counts."""
        from oracle import binding
        n = 2 * self.slots
        logn = self.log_slots + 1
        mods = binding.coeff_modulus_create(n, [60, 40, 40, 60])
        steps = [i for i in range(1, 16)] + [2 ** i for i in range(4, self.log_slots)]
        elts = binding.elts_from_steps(steps, n)
        o = binding.Oracle(logn, mods, 1, elts)
        rng = np.random.default_rng(0)
        seed = lambda k=1: rng.integers(0, 256, 64 * k, dtype=np.uint8)
        sk = o.gen_sk(seed())
        pk = o.gen_pk(sk, seed(), seed())
        rlk = o.gen_ksk(sk, o.sk_square(sk), seed(6))
        glk0 = o.gen_ksk(sk, o.galois(0, sk), seed(6))
        v = rng.normal(0, 1e-2, self.slots)
        t0 = time.perf_counter()
        ct1 = o.encrypt_asym(pk, o.encode(3, v, 2.0 ** 40, sparse_slots=self.slots), seed(), seed())
        t_enc = time.perf_counter() - t0
        ct2 = o.encrypt_asym(pk, o.encode(3, v * 0.5, 2.0 ** 40, sparse_slots=self.slots), seed(), seed())
        t0 = time.perf_counter()
        acc = o.square(3, o.poly_op("sub", 3, ct2, ct1).reshape(2, 3, n))
        acc = o.poly_op("add", 3, acc, acc)
        t_acc = time.perf_counter() - t0
        t0 = time.perf_counter()
        s = o.rescale(3, o.relinearize(3, acc, rlk))
        t_relin = time.perf_counter() - t0
        t0 = time.perf_counter()
        r = o.rotate(2, s, 0, glk0)
        t_rot = time.perf_counter() - t0
        pairs = self.n_clients * (self.n_clients - 1) // 2
        n_rot = 15 + (self.log_slots - 4)
        est = self.n_clients * self.chunks * t_enc + pairs * self.chunks * t_acc + pairs * (t_relin + n_rot * t_rot)
        sample = ("extrapolated from 1 encode+encrypt (%.3f s), 1 chunk sub+square+add (%.4f s), 1 relinearize+rescale (%.3f s), "
                  "1 rotation (%.3f s) x (%d ciphertexts, %d pair-chunks, %d pairs, %d rotations per pair)"
                  % (t_enc, t_acc, t_relin, t_rot, self.n_clients * self.chunks, pairs * self.chunks, pairs, n_rot))
        return est, sample


class HmultWorkload:
    """BASELINE configs[2] flavour: ciphertext multiply + relinearize + rescale at N = 2^16, L = 24,
    dnum = 3 (8 special primes), on seeded uniform ciphertexts with real keys."""
    name = "hmult"
    metric = "hmult_relin_rescale_ops_per_s"
    unit = "ops/s"
    higher_is_better = True
    dtype = "u64"
    scaling = "weak"

    def __init__(self, batch=8):
        self.batch = int(batch)
        self.logn, self.N, self.L, self.P = 16, 1 << 16, 24, 8
        self.launches_per_step = 0

    def bits(self):
        return [60] + [50] * 23 + [60] * 8

    def config(self):
        return {"workload": "C3 multiply+relinearize+rescale, N=2^16, L=24, dnum=3 (alpha=8), %d ciphertext pairs per step" % self.batch,
                "l2": "one ciphertext is 24 MiB, the relinearization key 96 MiB; a step streams far more than the 126 MB L2"}

    def setup_gpu(self, device):
        import torch
        from . import cabi
        self.torch = torch
        mods = cabi.coeff_modulus_create(self.N, self.bits())
        self.ctx = cabi.Context(self.logn, mods, self.P, device=device)
        rng = np.random.default_rng(5)
        seed = lambda k=1: rng.integers(0, 256, 64 * k, dtype=np.uint8)
        sk = self.ctx.gen_secret_key(seed())
        self.rlk = self.ctx.gen_switch_key(sk, self.ctx.multiply_poly_qp(sk, sk), seed(6))
        g = torch.Generator(device="cuda:%d" % device)
        g.manual_seed(9)
        shape = (self.batch, 2, self.L, self.N)
        self.a = torch.randint(0, 1 << 49, shape, dtype=torch.int64, device="cuda:%d" % device, generator=g)
        self.b = torch.randint(0, 1 << 49, shape, dtype=torch.int64, device="cuda:%d" % device, generator=g)
        self.ha = torch.empty(shape, dtype=torch.int64).pin_memory()
        self.hb = torch.empty(shape, dtype=torch.int64).pin_memory()
        self.ha.copy_(self.a)
        self.hb.copy_(self.b)
        self.hout = torch.empty((self.batch, 2, self.L - 1, self.N), dtype=torch.int64).pin_memory()
        self.out = None

    def step_gpu(self):
        l0 = _launches()
        ct3 = self.ctx.multiply(self.L, self.a, self.b, batch=self.batch)
        self.ctx.relinearize_batch(self.L, ct3, self.rlk)
        self.out = self.ctx.rescale_strided(self.L, ct3, self.batch, 2, 3 * self.L * self.N)
        self.launches_per_step = _launches() - l0

    def step_e2e(self):
        self.a.copy_(self.ha, non_blocking=True)
        self.b.copy_(self.hb, non_blocking=True)
        self.step_gpu()
        self.hout.copy_(self.out, non_blocking=True)
        return 2 * self.ha.numel() * 8, self.hout.numel() * 8

    def check_gpu(self):
        # linearity of the chain in its first argument: f(a, b) + f(a', b) = f(a + a', b) up to the
        # rescale's floor, so only a cheap sanity value is checked here; bit-exact parity lives in tests/
        return self.out is not None and bool((self.out >= 0).all())

    def units_per_step(self):
        return float(self.batch)

    def algorithmic_bytes_per_step(self):
        n, L, P, beta = self.N, self.L, self.P, 3
        tensor = 56 * L * n
        ks = 8 * n * (5 * L + 2 * beta * (L + P))
        resc = 2 * (L + L - 1) * n * 8
        return self.batch * (tensor + ks + resc)

    def time_dominant_kernel(self, timed):
        """the forward transform over as many limbs as one step's mod-up digits (beta x (L+P) per ciphertext),
        the kernel with the largest share of a key switch"""
        rows = self.batch * 3 * (self.L + self.P)
        buf = self.torch.randint(0, 1 << 49, (rows, self.N), dtype=self.torch.int64, device=self.a.device)
        groups = rows // (self.L + self.P)
        fn = lambda: self.ctx.ntt_forward(buf, groups, self.L, self.P)
        for _ in range(3):
            fn()
        ms, _ = timed(fn, 10)
        self._kernel_bytes = 16 * self.N * rows
        return ms / 10, "ntt_fwd_fixed_kernel<3> (plain input)"

    def roofline_kernel_bytes(self):
        return self._kernel_bytes

    def cpu_sample(self, threads):
        from oracle import binding
        mods = binding.coeff_modulus_create(self.N, self.bits())
        o = binding.Oracle(self.logn, mods, self.P, [])
        rng = np.random.default_rng(1)
        seed = lambda k=1: rng.integers(0, 256, 64 * k, dtype=np.uint8)
        sk = o.gen_sk(seed())
        rlk = o.gen_ksk(sk, o.sk_square(sk), seed(6))
        a = rng.integers(0, 1 << 49, (2, self.L, self.N), dtype=np.uint64)
        b = rng.integers(0, 1 << 49, (2, self.L, self.N), dtype=np.uint64)
        t0 = time.perf_counter()
        reps = 0
        while reps < 1 or time.perf_counter() - t0 < 5.0:
            o.rescale(self.L, o.relinearize(self.L, o.tensor(self.L, a, b), rlk))
            reps += 1
        dt = time.perf_counter() - t0
        return reps / dt, "%d x multiply+relinearize+rescale of one ciphertext pair" % reps


WORKLOADS = {"krum": KrumWorkload, "hmult": HmultWorkload}
