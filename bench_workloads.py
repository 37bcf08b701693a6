"""Workloads of bench.py: the encrypted-Krum distance round (the headline), the multiply + relinearize +
rescale chain at N = 2^16, L = 24, and the batched NTT / INTT sweep.

Each class follows the small protocol bench.py drives: setup_gpu / step_gpu / step_e2e / check_gpu /
cpu_sample, plus the bookkeeping the JSON line needs.  Inputs are seeded synthetic tensors with the shapes and
value distributions of the benchmark configurations (no dataset exists here).  Nothing at module level imports
torch or the CUDA library, so that the CPU arm (``--impl reference``) runs without either; the GPU legs import
them inside ``setup_gpu``.  The CPU checker under oracle/ is used in two places only: ``cpu_sample`` (the timed
CPU baseline) and ``check_gpu`` of the multiply chain (it is the checker there, never the thing measured)."""
import os
import time

import numpy as np

KRUM_BITS = [60, 40, 40, 60]
WIDE_BITS = [60] + [50] * 23 + [60] * 8

# DRAM traffic of one captured launch (ncu, dram__bytes_read.sum + dram__bytes_write.sum) beside the algorithmic
# bytes of that same launch; the summary each pair comes from is named.  bench.py scales a kernel's algorithmic
# bytes by this ratio for "traffic"; a kernel without a capture reports null.
NCU_TRAFFIC = {
    # mod-down transform of 128 encryptions, N = 2^16: 750.1 MB read + 386.7 MB written
    "ntt_fwd_kernel(fused input)": {"dram_bytes": 1136815360, "algorithmic_bytes": 1149239296,
                                    "summary": "profiles/ntt_fwd_fused_encrypt_batch128.md"},
    # <2,2> tile of the 10-client round, N = 2^15: 641.8 MB read + 11.9 MB written
    "krum_tile_kernel": {"dram_bytes": 653734400, "algorithmic_bytes": 651165696, "summary": "profiles/krum_tile_kernel_c4.md"},
}


def _oracle(threads):
    """the CPU checker with its OpenMP runtime set to ``threads`` (the variable must be set before the load)"""
    os.environ["OMP_NUM_THREADS"] = str(threads)
    from oracle import binding

    binding.set_threads(threads)
    return binding


def _launches():
    from lancelot_b200 import cabi

    return cabi.launch_count()


class KrumWorkload:
    """Encrypted Krum, distance phase: context + keys, encode + encrypt of every client, fused pair accumulation,
    batched relinearize / rescale / rotate-and-sum, gather of the score ciphertexts, per-client sums, decryption,
    argsort.  Default: 20 clients, N = 2^16 (ResNet-18 scale); --batch 10: 10 clients, N = 2^15 (MNIST-CNN scale)."""
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
        # how several GPUs share a round (EncryptedKrum.round): "chunks" or "p2p"
        self.exchange = os.environ.get("LANCELOT_KRUM_EXCHANGE", "chunks")

    def config(self):
        return {"workload": "%s encrypted Krum distance round: %d clients x %d float32, N=2^%d, %d ciphertexts per client, "
                            "%d pairs, chain {60,40,40|60}, scale 2^40" % (self.tag, self.n_clients, self.dim, self.log_slots + 1,
                                                                          self.chunks, self.n_clients * (self.n_clients - 1) // 2),
                "l2": "inputs (%.1f GiB of ciphertext) exceed the 126 MB L2" % (self.n_clients * self.chunks * 6 * (2 * self.slots) * 8 / 2 ** 30),
                "includes": "context + key generation, encode, encrypt, pair distances, score gather, decrypt, argsort",
                "excludes": "mask multiplication phase (GPU_mul_mask_weight)",
                "multi_gpu": "chunk axis sharded over the ranks, reduce-scatter of the partial pair sums" if self.exchange == "chunks"
                else "pairs sharded over the ranks, point-to-point exchange of client ciphertexts"}

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
        from lancelot_b200 import krum
        t0 = time.perf_counter()
        l0 = _launches()
        ek = krum.EncryptedKrum(log_slots=self.log_slots, device=self.device, seed=1, rank=self.rank, world_size=self.world)
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
        # the round takes the pinned host tensor itself: it copies one group of clients ahead of the encryption
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

    # -- pair tile alone ---------------------------------------------------------------------------------
    def time_pair_tile(self, timed):
        """the 2 x 4 pair tile (eight pair sums from six clients) on full-length clients, timed alone"""
        from lancelot_b200 import krum
        ek = krum.EncryptedKrum(log_slots=self.log_slots, device=self.device, seed=1)
        lb, N = ek.lb, ek.N
        cl = [ek.encrypt_client(self.updates[i], client=i) for i in range(6)]
        outs = [lb.empty(3, 3, N) for _ in range(8)]
        tile = lambda: lb.krum_accumulate_tile(3, cl[:2], cl[2:], outs)
        for _ in range(2):
            tile()
        tms, _ = timed(tile, 5)
        tile_bytes = 6 * cl[0].numel() * 8 + 8 * outs[0].numel() * 8
        return {"kernel": "krum_tile_kernel<2,4>", "bound": "hbm", "achieved": tile_bytes / (tms / 5 * 1e-3) / 1e9, "unit": "GB/s",
                "bytes_per_launch": tile_bytes, "pairs_per_launch": 8}

    def butterfly_roofs(self):
        """arithmetic ceilings of the transform for this chain's primes, as transform traffic (GB/s): the register-only
        butterfly rate of the 60-bit primes' variant and of the 40-bit primes' variant, and their harmonic mean"""
        from lancelot_b200 import krum
        ek = krum.EncryptedKrum(log_slots=self.log_slots, device=self.device, seed=1)
        n = ek.N
        per_limb = (n // 2) * (self.log_slots + 1)
        roofs = [ek.lb.butterfly_rate(v) / per_limb * 16 * n / 1e9 for v in (0, 3)]
        return {"int_strict_60bit": roofs[0], "fp64_40bit": roofs[1], "chain_mean": 2.0 / (1.0 / roofs[0] + 1.0 / roofs[1])}

    # -- CPU baseline -----------------------------------------------------------------------------------
    def cpu_sample(self, threads):
        """The CPU checker on a bounded sample: ``threads`` ciphertexts encoded + encrypted at once (one per core),
        as many pair-chunks (sub, square, add), as many pairs relinearized + rescaled and rotated once.  A round's
        time follows from the operation counts: every client encrypted once, as this library does it."""
        binding = _oracle(threads)
        n = 2 * self.slots
        logn = self.log_slots + 1
        mods = binding.coeff_modulus_create(n, KRUM_BITS)
        elts = binding.elts_from_steps([1], n)
        o = binding.Oracle(logn, mods, 1, elts)
        rng = np.random.default_rng(0)
        seed = lambda k=1: rng.integers(0, 256, 64 * k, dtype=np.uint8)
        sk = o.gen_sk(seed())
        pk = o.gen_pk(sk, seed(), seed())
        rlk = o.gen_ksk(sk, o.sk_square(sk), seed(6))
        glk0 = o.gen_ksk(sk, o.galois(0, sk), seed(6))
        b = max(int(threads), 1)
        vals = rng.normal(0, 1e-2, (2 * b, self.slots))
        seeds = seed(4 * b)
        o.encode_encrypt_batch(pk, vals[:2], 2.0 ** 40, seeds[:256])  # warm-up: page in tables and code
        t0 = time.perf_counter()
        cts = o.encode_encrypt_batch(pk, vals, 2.0 ** 40, seeds)
        t_enc = (time.perf_counter() - t0) / (2 * b)
        x, y = np.ascontiguousarray(cts[:b]), np.ascontiguousarray(cts[b:])
        acc = np.zeros((b, 3, 3, n), dtype=np.uint64)
        reps = 4
        t0 = time.perf_counter()
        for _ in range(reps):
            o.pair_chunk_batch(3, x, y, acc)
        t_acc = (time.perf_counter() - t0) / (reps * b)
        t0 = time.perf_counter()
        s = o.relin_rescale_batch(3, acc, rlk)
        t_relin = (time.perf_counter() - t0) / b
        t0 = time.perf_counter()
        o.rotate_batch(2, s, 0, glk0)
        t_rot = (time.perf_counter() - t0) / b
        pairs = self.n_clients * (self.n_clients - 1) // 2
        n_rot = 15 + (self.log_slots - 4)
        est = self.n_clients * self.chunks * t_enc + pairs * self.chunks * t_acc + pairs * (t_relin + n_rot * t_rot)
        sample = ("%d threads, one item per thread: %d encode+encrypt (%.4f s each amortised), %d pair-chunks sub+square+add (%.5f s), "
                  "%d relinearize+rescale (%.4f s), %d rotations (%.4f s); round = counts x amortised times "
                  "(%d ciphertexts, %d pair-chunks, %d pairs, %d rotations per pair)"
                  % (binding.max_threads(), 2 * b, t_enc, reps * b, t_acc, b, t_relin, b, t_rot, self.n_clients * self.chunks,
                     pairs * self.chunks, pairs, n_rot))
        return est, sample, binding.max_threads()


class HmultWorkload:
    """Ciphertext multiply + relinearize + rescale at N = 2^16, L = 24, dnum = 3 (8 special primes), on seeded uniform
    ciphertexts with real keys."""
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

    def config(self):
        return {"workload": "C3 multiply+relinearize+rescale, N=2^16, L=24, dnum=3 (alpha=8), %d ciphertext pairs per step" % self.batch,
                "l2": "one ciphertext is 24 MiB, the relinearization key 96 MiB; a step streams far more than the 126 MB L2"}

    def setup_gpu(self, device):
        import torch
        from lancelot_b200 import cabi
        self.torch = torch
        self.mods = cabi.coeff_modulus_create(self.N, WIDE_BITS)
        self.ctx = cabi.Context(self.logn, self.mods, self.P, device=device)
        rng = np.random.default_rng(5)
        seed = lambda k=1: rng.integers(0, 256, 64 * k, dtype=np.uint8)
        self.key_seeds = (seed(), seed(6))
        sk = self.ctx.gen_secret_key(self.key_seeds[0])
        self.rlk = self.ctx.gen_switch_key(sk, self.ctx.multiply_poly_qp(sk, sk), self.key_seeds[1])
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
        """the last ciphertext of the batch against the CPU checker, bit for bit (same keys from the same seeds)"""
        if self.out is None:
            return False
        from oracle import binding
        o = binding.Oracle(self.logn, self.mods, self.P, [])
        sk = o.gen_sk(self.key_seeds[0])
        rlk = o.gen_ksk(sk, o.sk_square(sk), self.key_seeds[1])
        k = self.batch - 1
        a = self.ha[k].numpy().view(np.uint64)
        b = self.hb[k].numpy().view(np.uint64)
        want = o.rescale(self.L, o.relinearize(self.L, o.tensor(self.L, a, b), rlk))
        got = self.out[k].cpu().numpy().view(np.uint64)
        return bool(np.array_equal(got.reshape(-1), want.reshape(-1)))

    def units_per_step(self):
        return float(self.batch)

    def algorithmic_bytes_per_step(self):
        n, L, P, beta = self.N, self.L, self.P, 3
        tensor = 56 * L * n
        ks = 8 * n * (5 * L + 2 * beta * (L + P))
        resc = 2 * (L + L - 1) * n * 8
        return self.batch * (tensor + ks + resc)

    def cpu_sample(self, threads):
        binding = _oracle(threads)
        mods = binding.coeff_modulus_create(self.N, WIDE_BITS)
        o = binding.Oracle(self.logn, mods, self.P, [])
        rng = np.random.default_rng(1)
        seed = lambda k=1: rng.integers(0, 256, 64 * k, dtype=np.uint8)
        sk = o.gen_sk(seed())
        rlk = o.gen_ksk(sk, o.sk_square(sk), seed(6))
        b = max(int(threads), 1)
        a = rng.integers(0, 1 << 49, (b, 2, self.L, self.N), dtype=np.uint64)
        c = rng.integers(0, 1 << 49, (b, 2, self.L, self.N), dtype=np.uint64)
        o.hmult_batch(self.L, a[:1], c[:1], rlk)
        t0 = time.perf_counter()
        reps = 0
        while reps < 1 or time.perf_counter() - t0 < 4.0:
            o.hmult_batch(self.L, a, c, rlk)
            reps += 1
        dt = time.perf_counter() - t0
        return reps * b / dt, "%d x %d concurrent multiply+relinearize+rescale (one per thread)" % (reps, b), binding.max_threads()


class NttWorkload:
    """Batched NTT/INTT sweep at N = 2^16 over 24 fifty-bit primes."""
    name = "ntt"
    metric = "ntt_hbm_gbs"
    unit = "GB/s"
    higher_is_better = True
    dtype = "u64"
    scaling = "weak"

    def __init__(self, batch=128, logn=16, limbs=24):
        self.batch, self.logn, self.limbs = int(batch), logn, limbs
        self.N = 1 << logn
        self.launches_per_step = 2

    def config(self):
        return {"workload": "C2 batched NTT+INTT, N=2^16, 24 x 50-bit primes, %d polynomials per step" % self.batch,
                "l2": "inputs (%.1f GiB per step) exceed the 126 MB L2" % (self.batch * self.limbs * self.N * 8 / 2 ** 30)}

    def algorithmic_bytes_per_step(self):
        # 16 bytes per coefficient per transform, forward + inverse
        return 2 * 16 * self.N * self.limbs * self.batch

    def setup_gpu(self, device):
        import torch
        from lancelot_b200 import cabi
        self.torch = torch
        self.ctx = cabi.Context(self.logn, cabi.coeff_modulus_create(self.N, [50] * self.limbs), 0, device=device)
        g = torch.Generator(device="cuda:%d" % device)
        g.manual_seed(1234)
        # residues uniform below 2^49 < q_i for every 50-bit prime
        self.data = torch.randint(0, 1 << 49, (self.batch, self.limbs, self.N), dtype=torch.int64, device="cuda:%d" % device, generator=g)
        self.orig = self.data.clone()
        self.host = torch.empty_like(self.data, device="cpu").pin_memory()
        self.host.copy_(self.data)
        self.host_out = torch.empty_like(self.host).pin_memory()

    def step_gpu(self):
        self.ctx.ntt_forward(self.data, self.batch, self.limbs, 0)
        self.ctx.ntt_inverse(self.data, self.batch, self.limbs, 0)

    def step_e2e(self):
        self.data.copy_(self.host, non_blocking=True)
        self.step_gpu()
        self.host_out.copy_(self.data, non_blocking=True)
        return self.host.numel() * 8, self.host_out.numel() * 8

    def check_gpu(self):
        return bool(self.torch.equal(self.data, self.orig))

    def units_per_step(self):
        return self.algorithmic_bytes_per_step() / 1e9  # GB

    def butterfly_roofs(self):
        """arithmetic ceiling of the transform: the register-only butterfly rate converted to transform traffic"""
        per_limb = (self.N // 2) * self.logn
        to_gbs = lambda rate: rate / per_limb * 16 * self.N / 1e9
        names = ["int_strict", "int_lazy", "fp64_50bit", "fp64_40bit"]
        out = {n: to_gbs(self.ctx.butterfly_rate(i)) for i, n in enumerate(names)}
        out["this_workload"] = to_gbs(self.ctx.butterfly_rate())  # the variant this workload's primes take
        return out

    def cpu_sample(self, threads):
        """forward + inverse of ``threads`` polynomials (24 limbs each), one limb per thread at a time"""
        binding = _oracle(threads)
        o = binding.Oracle(self.logn, binding.coeff_modulus_create(self.N, [50] * self.limbs), 0)
        rng = np.random.default_rng(0)
        b = max(int(threads) // 4, 1)
        data = rng.integers(0, 1 << 49, (b, self.limbs, self.N), dtype=np.uint64)
        orig = data.copy()
        o.ntt_roundtrip_batch(data, self.limbs)
        reps = 0
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < 3.0 or reps < 2:
            o.ntt_roundtrip_batch(data, self.limbs)
            reps += 1
        dt = time.perf_counter() - t0
        assert np.array_equal(data, orig)
        gb = reps * b * 2 * 16 * self.N * self.limbs / 1e9
        return gb / dt, "%d x (NTT+INTT of %d polynomials, 24 limbs each)" % (reps, b), binding.max_threads()


class MaskWorkload:
    """The aggregation phase of encrypted Krum (GPU_mul_mask_weight, lancelot-main-GPU/utils/byzantine_fl.py:371-429) on
    the 20-client round's ciphertexts: every client's ciphertexts times its encrypted mask (Enc(1/k) for the k selected
    clients, Enc(0) for the others), summed per chunk, size-3 decryption, decoding, gather of the averaged update.
    The ciphertexts are where the distance round left them: each rank holds its chunk range of every client."""
    name = "mask"
    metric = "encrypted_mask_multiplication_s"
    unit = "s"
    higher_is_better = False
    dtype = "u64"
    scaling = "strong"

    def __init__(self, batch=20):
        self.n_clients = int(batch)
        self.dim, self.log_slots = (1663370, 14) if self.n_clients == 10 else (11173962, 15)
        self.slots = 1 << self.log_slots
        self.chunks = (self.dim + self.slots - 1) // self.slots
        self.launches_per_step = 0
        self.selected = [3, 7, 11]  # a 3-hot mask with 1/3: the encrypted trimmed mean of three clients

    def config(self):
        return {"workload": "mask multiplication over %d clients x %d ciphertexts, N=2^%d, mask of %d clients, decrypt + decode of %d chunks"
                            % (self.n_clients, self.chunks, self.log_slots + 1, len(self.selected), self.chunks),
                "l2": "inputs (%.1f GiB of ciphertext) exceed the 126 MB L2" % (self.n_clients * self.chunks * 6 * (2 * self.slots) * 8 / 2 ** 30),
                "includes": "mask encryption, ct x ct products and sums, size-3 decryption, decoding, gather of the result",
                "excludes": "encryption of the clients' updates (done by the distance round)"}

    def algorithmic_bytes_per_step(self):
        # every client ciphertext read once, one size-3 ciphertext per chunk written and read again by the decryption
        return self.chunks * (2 * self.slots) * 3 * 8 * (2 * self.n_clients + 2 * 3)

    def setup_gpu(self, device):
        import torch
        import torch.distributed as dist
        from lancelot_b200 import krum
        self.torch = torch
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.ek = krum.EncryptedKrum(log_slots=self.log_slots, device=device, seed=1)
        g = torch.Generator(device="cuda:%d" % device)
        g.manual_seed(20240)
        self.updates = torch.randn(self.n_clients, self.dim, generator=g, device="cuda:%d" % device, dtype=torch.float32) * 1e-2
        lo, hi = krum.chunk_range(self.chunks, self.rank, self.world)
        self.cts = self.ek.encrypt_slices(self.updates, lo, hi)
        self.want = self.updates[self.selected].double().mean(dim=0)
        self.hout = torch.empty(self.dim, dtype=torch.float64).pin_memory()
        self.out = None

    def step_gpu(self):
        l0 = _launches()
        self.kept = {}
        self.out = self.ek.aggregate_sharded(self.cts, self.selected, self.dim, self.rank, self.world, keep=self.kept)
        self.launches_per_step = _launches() - l0

    def step_e2e(self):
        # the ciphertexts are produced on the device by the distance round; the host hands over the selection and
        # reads the averaged update back
        self.step_gpu()
        self.hout.copy_(self.out, non_blocking=True)
        return 8 * len(self.selected), self.hout.numel() * 8

    def check_gpu(self):
        """the first chunk's size-3 sum against the CPU checker, bit for bit; the decoded average against the float64
        mean of the selected updates (the error is the encryption noise of 2^16-coefficient ciphertexts over the
        scale 2^40, a few 1e-7 on values of 1e-2: the bar is 1e-5 absolute)"""
        from oracle import binding
        self.abs_err = float((self.out - self.want).abs().max())
        o = binding.Oracle(self.log_slots + 1, self.ek.context.moduli, 1, [])
        masks = self.kept["masks"].cpu().numpy().view(np.uint64)
        want = np.zeros((3, 3, 2 * self.slots), dtype=np.uint64)
        for k in range(self.n_clients):
            ct = self.cts[k][0].cpu().numpy().view(np.uint64)
            want = o.poly_op("add", 3, want, o.tensor(3, ct, masks[k]))
        got = self.kept["acc0"].cpu().numpy().view(np.uint64)
        self.bit_exact = bool(np.array_equal(got.reshape(-1), want.reshape(-1)))
        return bool(self.bit_exact and self.abs_err < 1e-5)

    def units_per_step(self):
        return 1.0

    def cpu_sample(self, threads):
        binding = _oracle(threads)
        n = 2 * self.slots
        o = binding.Oracle(self.log_slots + 1, binding.coeff_modulus_create(n, KRUM_BITS), 1, [])
        rng = np.random.default_rng(0)
        b = max(int(threads), 1)
        mods = o.moduli
        x = np.stack([rng.integers(0, mods[r % 3], n, dtype=np.uint64) for r in range(b * 6)]).reshape(b, 2, 3, n)
        mask = np.ascontiguousarray(x[0])
        acc = np.zeros((b, 3, 3, n), dtype=np.uint64)
        sk = o.gen_sk(rng.integers(0, 256, 64, dtype=np.uint8))
        o.mask_chunk_batch(3, x, mask, acc)
        reps = 3
        t0 = time.perf_counter()
        for _ in range(reps):
            o.mask_chunk_batch(3, x, mask, acc)
        t_mul = (time.perf_counter() - t0) / (reps * b)
        t0 = time.perf_counter()
        pt = o.decrypt(3, acc[0], sk)
        o.decode(3, pt, 2.0 ** 80, self.slots)
        t_dec = time.perf_counter() - t0  # single ciphertext, limb-parallel
        est = self.n_clients * self.chunks * t_mul + self.chunks * t_dec / max(1, min(b, 3))
        return est, ("%d threads: %d ct x mask products + adds (%.5f s each amortised), 1 size-3 decrypt + decode (%.4f s); phase = "
                     "%d products + %d decryptions" % (binding.max_threads(), reps * b, t_mul, t_dec, self.n_clients * self.chunks, self.chunks)), binding.max_threads()


class EncryptWorkload:
    """Fused encode + public-key encryption of float32 chunks at the 20-client round's parameters (N = 2^16, chain
    {60,40,40|60}, 32768 slots): the phase that takes the largest share of a round, as a component benchmark and as the
    small case for profiler captures of its kernels."""
    name = "encrypt"
    metric = "encode_encrypt_ciphertexts_per_s"
    unit = "ciphertexts/s"
    higher_is_better = True
    dtype = "u64"
    scaling = "weak"

    def __init__(self, batch=342):
        self.batch = int(batch)
        self.log_slots = 15
        self.slots = 1 << self.log_slots
        self.launches_per_step = 0

    def config(self):
        return {"workload": "encode + encrypt of %d chunks of 32768 float32, N=2^16, chain {60,40,40|60}, scale 2^40" % self.batch,
                "l2": "scratch and output of one call (%.2f GiB) exceed the 126 MB L2" % (self.batch * 27 * 2 * self.slots * 8 / 2 ** 30)}

    def algorithmic_bytes_per_step(self):
        # values in, ciphertext out; everything between is scratch
        return self.batch * (self.slots * 4 + 6 * 2 * self.slots * 8)

    def setup_gpu(self, device):
        import torch
        from lancelot_b200 import krum
        self.torch = torch
        self.ek = krum.EncryptedKrum(log_slots=self.log_slots, device=device, seed=1, encrypt_batch=max(self.batch, 64))
        g = torch.Generator(device="cuda:%d" % device)
        g.manual_seed(4)
        self.vals = torch.randn(self.batch, self.slots, generator=g, device="cuda:%d" % device, dtype=torch.float32) * 1e-2
        self.host = torch.empty(self.vals.shape, dtype=torch.float32).pin_memory()
        self.host.copy_(self.vals)
        self.seeds = self.ek.client_seeds(0, self.batch)
        self.out = self.ek.lb.empty(self.batch, 2, 3, self.ek.N)
        self.hout = torch.empty((2, 3, self.ek.N), dtype=torch.int64).pin_memory()

    def step_gpu(self):
        l0 = _launches()
        self.ek.encrypt_chunks(self.vals, self.seeds, out=self.out)
        self.launches_per_step = _launches() - l0

    def step_e2e(self):
        self.vals.copy_(self.host, non_blocking=True)
        self.step_gpu()
        self.hout.copy_(self.out[-1], non_blocking=True)  # the ciphertexts stay on the device; one is read back
        return self.host.numel() * 4, self.hout.numel() * 8

    def check_gpu(self):
        """the last ciphertext against the CPU checker, bit for bit (same keys and seeds)"""
        from oracle import binding
        ek = self.ek
        o = binding.Oracle(self.log_slots + 1, ek.context.moduli, 1, [])
        pk = ek.pk.data.cpu().numpy().view(np.uint64)
        k = self.batch - 1
        v = self.host[k].numpy().astype(np.float64)
        want = o.encrypt_asym(pk, o.encode(3, v, ek.scale, sparse_slots=self.slots), self.seeds[128 * k:128 * k + 64], self.seeds[128 * k + 64:128 * k + 128])
        got = self.out[k].cpu().numpy().view(np.uint64)
        return bool(np.array_equal(got.reshape(-1), want.reshape(-1)))

    def units_per_step(self):
        return float(self.batch)

    def cpu_sample(self, threads):
        binding = _oracle(threads)
        n = 2 * self.slots
        o = binding.Oracle(self.log_slots + 1, binding.coeff_modulus_create(n, KRUM_BITS), 1, [])
        rng = np.random.default_rng(0)
        seed = lambda k=1: rng.integers(0, 256, 64 * k, dtype=np.uint8)
        sk = o.gen_sk(seed())
        pk = o.gen_pk(sk, seed(), seed())
        b = 2 * max(int(threads), 1)
        vals = rng.normal(0, 1e-2, (b, self.slots))
        seeds = seed(2 * b)
        o.encode_encrypt_batch(pk, vals[:2], 2.0 ** 40, seeds[:256])
        t0 = time.perf_counter()
        o.encode_encrypt_batch(pk, vals, 2.0 ** 40, seeds)
        dt = time.perf_counter() - t0
        return b / dt, "%d encode+encrypt, one per thread at a time" % b, binding.max_threads()


WORKLOADS = {"krum": KrumWorkload, "hmult": HmultWorkload, "ntt": NttWorkload, "encrypt": EncryptWorkload, "mask": MaskWorkload}
