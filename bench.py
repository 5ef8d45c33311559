#!/usr/bin/env python
"""Benchmark of the RNS-CKKS evaluation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload hrot|hmult|ntt] [--impl reference]

One "step" is one pass of the hot path over one batch of synthetic, seeded input that is
already resident in HBM:
  hrot   one homomorphic rotation with hybrid key switching, N=2^16, L=35 primes of 50 bits,
         K=5 extension primes of 60 bits, dnum=7 (uniform ciphertext limbs and key limbs);
         metric: key-switch ops/s                                            [default]
  hmult  one HMult + relinearise + rescale, L=24 (60-bit first prime, 50-bit rest), K=1, dnum=24
  ntt    forward + inverse NTT of 48 limbs x 8 polynomials of 50-bit primes
  hoisted  eight rotations of one ciphertext sharing one ModUp (HRot parameters); rotations/s
  bsgs   one 8 x 8 baby-step / giant-step multiply-accumulate (64 diagonals, HRot parameters)
With N > 1 ranks (torchrun) every rank runs the same workload on its own ciphertexts
(independent ciphertexts, no data-path collective): weak scaling, value = all ranks' ops / max
time over ranks.  For hrot the same operation is also timed limb-sharded over all ranks
(ciphertext and key split by RNS limb, one NCCL all-gather per key switch: the latency of one
operation, strong scaling) and reported under `limb_sharded`; `--parallelism limb` makes that
the headline instead.

Prints one JSON line.  `value` is device-resident throughput timed with CUDA events; `e2e` is the
same metric through the C ABI with host buffers (pinned), host->device and device->host copies
of every step inside the timed region (cerium_b200.host_pipeline overlaps upload, evaluation and
download of consecutive steps on three streams); `roofline` describes the dominant kernel pair (forward NTT) timed live
with CUDA events; `cpu_baseline` is the oracle (a port of the reference algorithm) on a bounded
sample on the host cores.  `--impl reference` times that CPU port alone.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from cerium_b200 import params  # noqa: E402

LOGN = 16
N = 1 << LOGN
# dram__bytes_read.sum + dram__bytes_write.sum of the forward-NTT launch pair from the ncu capture
# summarised in profiles/hrot_u64_top_kernels_ncu_full.md: 443.2 MB for 245 u64 limbs (traffic grows
# in proportion to the limbs transformed)
NTT_PAIR_DRAM_BYTES_PER_LIMB = 443.2e6 / 245
# what the CPU figure is: the checker, not a tuned evaluator
PORT_QUALITY = ("unoptimised checker: plain-C restatement with a 128-bit remainder in every modular product outside "
                "the transforms; a Barrett/Shoup CPU evaluator would be several times faster")


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


PROBE_NAMES = ("mad.lo.u32", "mad.wide.u32", "mul.hi.u64", "mul.lo.u64", "add.u64", "butterfly_u64_strict",
               "butterfly_u64_lazy", "butterfly_u32", "fma.rn.f64", "butterfly_u64_fp64")


def probe_int_pipe(device):
    """Register-only instruction / butterfly rates in Gop/s on `device` (the arithmetic roofline of
    the 64-bit kernels), from the bench-side probe library built next to the evaluation library."""
    import ctypes
    from cerium_b200 import build as cbuild
    dll = ctypes.CDLL(cbuild.PROBE_LIB)
    dll.cerium_probe_int_pipe.restype = ctypes.c_int
    dll.cerium_probe_int_pipe.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.c_int]
    dll.cerium_probe_last_error.restype = ctypes.c_char_p
    buf = (ctypes.c_double * 10)()
    if dll.cerium_probe_int_pipe(device, buf, 10) != 0:
        raise RuntimeError("probe: " + dll.cerium_probe_last_error().decode())
    return dict(zip(PROBE_NAMES, [float(v) for v in buf]))


class Watchdog:
    """Ends the process when the benchmark makes no progress for `limit_s` seconds (a collective whose peers never
    arrive would otherwise wait until the caller's own limit): the stage it was in goes to stderr, exit code 3."""

    def __init__(self, limit_s: float):
        self.limit_s = limit_s
        self.stage = "start"
        self.t = time.monotonic()
        self.done = False
        if limit_s > 0:
            threading.Thread(target=self._watch, daemon=True).start()

    def at(self, stage: str):
        self.stage = stage
        self.t = time.monotonic()

    def _watch(self):
        while not self.done:
            time.sleep(5)
            if time.monotonic() - self.t > self.limit_s:
                sys.stderr.write("bench.py: no progress for %d s in stage '%s' (rank %s); giving up\n"
                                 % (self.limit_s, self.stage, os.environ.get("RANK", "0")))
                sys.stderr.flush()
                os._exit(3)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,utilization.gpu,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark_start(self):
        """Samples taken before this call (idle GPU, start-up) are not part of the record."""
        self.t_start = time.perf_counter()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t_start = getattr(self, "t_start", 0.0)
        for ts, ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9 or ts < t_start:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------

class Workload:
    name = ""
    metric = ""
    unit = ""

    def setup(self, lib, torch, rank):
        raise NotImplementedError

    def step(self):
        raise NotImplementedError

    def fork(self):
        pass

    def join(self):
        pass

    def e2e_drain(self):
        if getattr(self, "pipe", None) is not None:
            self.pipe.drain()


def _rand_limbs_gpu(torch, moduli, prime_idx, lead, gen):
    """[lead..., len(prime_idx), N] int64 uniform residues on the GPU (seeded)."""
    q = torch.tensor([moduli[p] for p in prime_idx], dtype=torch.int64, device="cuda").view(-1, 1)
    shape = tuple(lead) + (len(prime_idx), N)
    x = torch.randint(0, 1 << 62, shape, dtype=torch.int64, device="cuda", generator=gen)
    return (x % q).contiguous()


class HRotWorkload(Workload):
    name = "hrot_N65536_L35_K5_dnum7_u64"
    metric = "hrot_keyswitch_ops_per_s"
    unit = "ops/s"
    ops_per_step = 1

    def __init__(self, n_cts=4):
        self.prm = params.config_hrot(LOGN, 35, 5, 7)
        self.n_cts = n_cts  # rotating set of ciphertexts so consecutive ops do not reuse inputs

    def setup(self, lib, torch, rank, world=1, sharded=False, comm=None, ext_split=True, inflight=1):
        from cerium_b200 import _capi
        self.torch = torch
        prm = self.prm
        self.sharded = sharded and world > 1
        self.rank, self.world = rank, world
        self.ctx = _capi.Context(lib, prm.moduli, 64, device=torch.cuda.current_device())
        all_idx = prm.q_idx + prm.p_idx
        if self.sharded:
            # every rank generates the SAME ciphertexts and key and keeps its own limbs (round robin by
            # limb); `inflight` operations are in flight at a time, each on a plan and a stream of its own,
            # so that one operation's exchange runs under another's arithmetic
            from cerium_b200 import sharded as sh
            self.sh = sh
            self.comm, self.ext_split, self.inflight = comm, ext_split, inflight
            gen = torch.Generator(device="cuda").manual_seed(0xCE210003)
            full_evk = _rand_limbs_gpu(torch, prm.moduli, all_idx, (prm.dnum, 2), gen)
            full_cts = [_rand_limbs_gpu(torch, prm.moduli, prm.q_idx, (2,), gen) for _ in range(self.n_cts)]
            self.mine = sh.local_limb_indices(prm.L, rank, world)
            self.evk = sh.shard_key(full_evk, prm.L, rank, world, ext_split)
            self.cts = [torch.stack([sh.shard_poly(c[0], rank, world), sh.shard_poly(c[1], rank, world)])
                        for c in full_cts]
            self.full_evk, self.full_ct0 = full_evk, full_cts[0]     # kept for verify(), dropped afterwards
            # a communicator per operation in flight: collectives of one communicator run in issue order,
            # so with one communicator an operation's second exchange would hold back the next operation's first
            self.comms = [comm] + [sh.nccl_comm(lib, rank, world, torch.cuda.current_device()) for _ in range(inflight - 1)]
            self.sks = [sh.ShardedKeySwitch(self.ctx, prm, c, _capi.BCONV_EXACT, _capi.ROUND_HALF, ext_split=ext_split)
                        for c in self.comms]
            self.streams = [torch.cuda.Stream() for _ in range(inflight)]
            self.outs = [torch.empty_like(self.cts[0]) for _ in range(max(self.n_cts, inflight))]
            k_loc = self.sks[0].k_local
            # iNTT pair, [gather], BConv, NTT pair, inner product, iNTT pair, [gather], BConv, SuD pair
            self.gpu_launches_per_step = 2 + 1 + 2 + 1 + (2 if k_loc else 0) + 1 + 2
        else:
            gen = torch.Generator(device="cuda").manual_seed(0xCE210003 + rank)
            # exact conversion + rounding: the semantics that are low-noise with 50/60-bit primes.
            # `inflight` independent operations may be in flight, each on a plan (workspace) and a stream
            # of its own: the latency-bound small launches of one then run beside the other's large ones
            self.inflight = max(1, inflight)
            self.kss = [_capi.KeySwitch(self.ctx, prm.q_idx, prm.p_idx, prm.dnum, _capi.BCONV_EXACT, _capi.ROUND_HALF)
                        for _ in range(self.inflight)]
            self.ks = self.kss[0]
            self.streams = [torch.cuda.Stream() for _ in range(self.inflight)] if self.inflight > 1 else []
            self.evk = _rand_limbs_gpu(torch, prm.moduli, all_idx, (prm.dnum, 2), gen)
            self.n_cts = self.inflight * -(-self.n_cts // self.inflight)   # a buffer is only ever used by one stream
            self.cts = [_rand_limbs_gpu(torch, prm.moduli, prm.q_idx, (2,), gen) for _ in range(self.n_cts)]
            self.outs = [torch.empty_like(self.cts[0]) for _ in range(self.n_cts)]
            # iNTT pair, BConv, NTT pair, inner product, iNTT pair, BConv, SuD pair (the rotation itself is
            # folded into the reads of the iNTT, the inner product and the SuD tail: no launch of its own)
            self.gpu_launches_per_step = 2 + 1 + 2 + 1 + 2 + 1 + 2
        self.elt = hrot_galois_elt()
        self.i = 0
        self.ct_bytes = self.cts[0].numel() * 8
        # algorithmic (compulsory) bytes of one HRot: ciphertext in + key + ciphertext out
        self.alg_bytes = (2 * prm.L + prm.dnum * 2 * (prm.L + prm.K) + 2 * prm.L) * N * 8
        self.host_ins = [torch.empty(self.cts[0].shape, dtype=torch.int64).pin_memory() for _ in range(3)]
        for h in self.host_ins:
            h.copy_(self.cts[0].cpu())

    def _hrot(self, ct, out, stream=None, slot=0):
        s = self.torch.cuda.current_stream().cuda_stream if stream is None else stream
        if self.sharded:
            self.sks[slot].hrot(out[0], out[1], ct[0], ct[1], self.evk, self.elt, s)
        else:
            self.kss[slot].hrot(out[0].data_ptr(), out[1].data_ptr(), ct[0].data_ptr(), ct[1].data_ptr(),
                                self.evk.data_ptr(), self.elt, s)

    def step(self):
        k = self.i % self.n_cts
        if self.streams:
            slot = self.i % self.inflight
            self._hrot(self.cts[k], self.outs[k if not self.sharded else slot], self.streams[slot].cuda_stream, slot)
        else:
            self._hrot(self.cts[k], self.outs[k])
        self.i += 1

    # the timed region is bracketed by events on the current stream: the side streams start after its
    # first event and are joined before its second
    def fork(self):
        cur = self.torch.cuda.current_stream()
        for st in self.streams:
            st.wait_stream(cur)

    def join(self):
        cur = self.torch.cuda.current_stream()
        for st in self.streams:
            cur.wait_stream(st)

    def verify(self, orc_mod):
        """One operation on the benchmark's own inputs, every limb bit for bit, outside the timed region.
        One GPU: against the oracle.  Sharded: every rank runs the whole one-GPU operation on the same
        ciphertext (the path the oracle pins at this shape) and compares its own limbs with it, for
        every plan in flight."""
        torch, prm = self.torch, self.prm
        u = lambda t: t.cpu().numpy().view(np.uint64)  # noqa: E731
        if self.sharded:
            from cerium_b200 import _capi
            ks = _capi.KeySwitch(self.ctx, prm.q_idx, prm.p_idx, prm.dnum, _capi.BCONV_EXACT, _capi.ROUND_HALF)
            full = torch.empty_like(self.full_ct0)
            ks.hrot(full[0].data_ptr(), full[1].data_ptr(), self.full_ct0[0].data_ptr(), self.full_ct0[1].data_ptr(),
                    self.full_evk.data_ptr(), self.elt, torch.cuda.current_stream().cuda_stream)
            ok = True
            for slot in range(self.inflight):
                out = self.outs[slot]
                out.zero_()
                self._hrot(self.cts[0], out, None, slot)
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(out, full[:, self.mine]))
            ks.close()
            del self.full_evk, self.full_ct0, full
            torch.cuda.empty_cache()
            return ok
        ct, out = self.cts[0], self.outs[0]
        self._hrot(ct, out)
        torch.cuda.synchronize()
        octx = orc_mod.OracleContext(LOGN, prm.moduli)
        w0, w1 = octx.hrot(orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, self.elt,
                           u(ct[0]), u(ct[1]), u(self.evk))
        got = u(out)
        return bool(np.array_equal(got[0], w0) and np.array_equal(got[1], w1))

    def e2e_step(self):
        if getattr(self, "pipe", None) is None:
            from cerium_b200.host_pipeline import HostPipeline

            def op(ins, outs, stream):
                self._hrot(ins[0], outs[0], stream, 0)
            self.pipe = HostPipeline(self.torch, [self.cts[0].shape], [self.cts[0].shape], op)
            self.e2e_i = 0
        self.pipe.submit([self.host_ins[self.e2e_i % len(self.host_ins)]])
        self.e2e_i += 1
        return self.pipe.in_bytes, self.pipe.out_bytes

    def e2e_drain(self):
        if getattr(self, "pipe", None) is not None:
            self.pipe.drain()

    # the collective(s) of one sharded operation alone, on buffers of the same size
    def collective_step(self):
        sk = self.sks[0]
        if not hasattr(self, "cbuf"):
            n_q = self.world * sk.g
            n_p = self.world * 2 * (-(-self.prm.K // self.world)) if self.ext_split else 0
            self.cbuf = self.torch.zeros((n_q + n_p, N), dtype=self.torch.int64, device="cuda")
            self.c_nq = n_q
        s = self.torch.cuda.current_stream().cuda_stream
        base = self.cbuf.data_ptr()
        self.comm.allgather_limbs(self.ctx, base, base + self.rank * sk.g * N * 8, sk.g, s)
        if self.ext_split:
            kg = 2 * (-(-self.prm.K // self.world))
            pb = base + self.c_nq * N * 8
            self.comm.allgather_limbs(self.ctx, pb, pb + self.rank * kg * N * 8, kg, s)

    # dominant kernel pair: forward NTT over the raised limbs (dnum*(L+K) - L limb transforms)
    def roofline_setup(self):
        prm = self.prm
        self.rl_idx = []
        if getattr(self, "sharded", False):
            mine = self.mine
            ext = [prm.p_idx[k] for k in self.sh.local_ext_indices(prm.L, prm.K, self.rank, self.world, self.ext_split)]
        else:
            mine = list(range(prm.L))
            ext = prm.p_idx
        for d in range(prm.dnum):
            for i in mine:
                if i % prm.dnum != d:
                    self.rl_idx.append(prm.q_idx[i])
            self.rl_idx.extend(ext)
        gen = self.torch.Generator(device="cuda").manual_seed(5)
        self.rl_buf = _rand_limbs_gpu(self.torch, prm.moduli, self.rl_idx, (), gen)
        self.rl_bytes = 2 * len(self.rl_idx) * N * 8  # read once + write once
        self.rl_name = "forward NTT (column pass + row pass), %d limbs u64" % len(self.rl_idx)

    def roofline_step(self):
        self.ctx.ntt_forward(self.rl_buf.data_ptr(), self.rl_buf.data_ptr(), self.rl_idx,
                             stream=self.torch.cuda.current_stream().cuda_stream)

    # CPU baseline: the oracle's HRot on the same parameter set (one op)
    def cpu_sample(self, orc_mod):
        prm = self.prm
        rng = np.random.default_rng(1)
        octx = orc_mod.OracleContext(LOGN, prm.moduli)
        all_idx = prm.q_idx + prm.p_idx

        def rl(idx, lead=()):
            return np.stack([rng.integers(0, prm.moduli[p], size=tuple(lead) + (N,), dtype=np.uint64) for p in idx])
        c0, c1 = rl(prm.q_idx), rl(prm.q_idx)
        evk = np.stack([np.stack([rl(all_idx) for _ in range(2)]) for _ in range(prm.dnum)])
        t0 = time.perf_counter()
        octx.hrot(orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, hrot_galois_elt(), c0, c1, evk)
        dt = time.perf_counter() - t0
        return 1.0 / dt, "1 HRot (L=35, K=5, dnum=7), oracle port with OpenMP over limbs"


def hrot_galois_elt():
    """Galois element 5^step mod 2N of the seeded rotation step in [1, 2^15)."""
    step = int(np.random.default_rng(0xCE210003).integers(1, 1 << 15))
    return pow(5, step, 2 * N)


class HMultWorkload(Workload):
    name = "hmult_relin_rescale_N65536_L24_K1_dnum24_u64"
    metric = "hmult_keyswitch_ops_per_s"
    unit = "ops/s"
    ops_per_step = 1

    # 2: the rescale is folded into the relinearisation's ModDown (one division by P * q_last, the way the
    # reference lowers a key switch with rescale levels); 1: ModDown, then rescale
    rescale_mode = 2

    def __init__(self):
        self.prm = params.config_hmult(LOGN, 24)
        self.rescale_mode = int(os.environ.get("CERIUM_BENCH_HMULT_RESCALE", self.rescale_mode))

    def setup(self, lib, torch, rank, world=1, sharded=False):
        from cerium_b200 import _capi
        self.torch = torch
        prm = self.prm
        self.ctx = _capi.Context(lib, prm.moduli, 64, device=torch.cuda.current_device())
        self.ks = _capi.KeySwitch(self.ctx, prm.q_idx, prm.p_idx, prm.dnum, _capi.BCONV_EXACT, _capi.ROUND_HALF)
        gen = torch.Generator(device="cuda").manual_seed(0xCE210001 + rank)
        all_idx = prm.q_idx + prm.p_idx
        self.evk = _rand_limbs_gpu(torch, prm.moduli, all_idx, (prm.dnum, 2), gen)
        self.a = _rand_limbs_gpu(torch, prm.moduli, prm.q_idx, (2,), gen)
        self.b = _rand_limbs_gpu(torch, prm.moduli, prm.q_idx, (2,), gen)
        self.out = torch.empty((2, prm.L - 1, N), dtype=torch.int64, device="cuda")
        self.alg_bytes = (4 * prm.L + prm.dnum * 2 * (prm.L + prm.K) + 2 * (prm.L - 1)) * N * 8
        self.host_in = torch.empty((2,) + tuple(self.a.shape), dtype=torch.int64).pin_memory()
        self.host_in[0].copy_(self.a.cpu())
        self.host_in[1].copy_(self.b.cpu())
        self.host_out = torch.empty(self.out.shape, dtype=torch.int64).pin_memory()
        # tensor; key switch: iNTT pair, NTT pair x2 (576 limbs in two batches), inner product, iNTT pair,
        # BConv, SuD pair; then either the rescale of both polynomials (iNTT pair, SuD pair) or, folded
        # into the ModDown, two PMU launches
        self.gpu_launches_per_step = 1 + (2 + 4 + 1 + 2 + 1 + 2) + (2 if self.rescale_mode == 2 else 4)

    def step(self):
        s = self.torch.cuda.current_stream().cuda_stream
        a, b, o = self.a, self.b, self.out
        self.ks.hmult(o[0].data_ptr(), o[1].data_ptr(), a[0].data_ptr(), a[1].data_ptr(), b[0].data_ptr(),
                      b[1].data_ptr(), self.evk.data_ptr(), self.rescale_mode, s)

    def verify(self, orc_mod):
        torch, prm = self.torch, self.prm
        self.step()
        torch.cuda.synchronize()
        u = lambda t: t.cpu().numpy().view(np.uint64)  # noqa: E731
        octx = orc_mod.OracleContext(LOGN, prm.moduli)
        args = (u(self.a[0]), u(self.a[1]), u(self.b[0]), u(self.b[1]), u(self.evk))
        if self.rescale_mode == 2:
            w0, w1 = octx.hmult_relin_fused(orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, *args)
        else:
            w0, w1 = octx.hmult_relin(orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF, True, prm.q_idx, prm.p_idx, prm.dnum, *args)
        got = u(self.out)
        return bool(np.array_equal(got[0], w0) and np.array_equal(got[1], w1))

    def e2e_step(self):
        if getattr(self, "pipe", None) is None:
            from cerium_b200.host_pipeline import HostPipeline

            def op(ins, outs, stream):
                a, b, o = ins[0], ins[1], outs[0]
                self.ks.hmult(o[0].data_ptr(), o[1].data_ptr(), a[0].data_ptr(), a[1].data_ptr(), b[0].data_ptr(),
                              b[1].data_ptr(), self.evk.data_ptr(), self.rescale_mode, stream)
            self.pipe = HostPipeline(self.torch, [self.a.shape, self.b.shape], [self.out.shape], op)
        self.pipe.submit([self.host_in[0], self.host_in[1]])
        return self.pipe.in_bytes, self.pipe.out_bytes

    def roofline_setup(self):
        prm = self.prm
        self.rl_idx = []
        for d in range(prm.dnum):
            for i, p in enumerate(prm.q_idx + prm.p_idx):
                if not (i < prm.L and i % prm.dnum == d):
                    self.rl_idx.append(p)
        gen = self.torch.Generator(device="cuda").manual_seed(5)
        self.rl_buf = _rand_limbs_gpu(self.torch, prm.moduli, self.rl_idx, (), gen)
        self.rl_bytes = 2 * len(self.rl_idx) * N * 8
        self.rl_name = "forward NTT (column pass + row pass), %d limbs u64" % len(self.rl_idx)

    def roofline_step(self):
        self.ctx.ntt_forward(self.rl_buf.data_ptr(), self.rl_buf.data_ptr(), self.rl_idx,
                             stream=self.torch.cuda.current_stream().cuda_stream)

    def cpu_sample(self, orc_mod):
        prm = self.prm
        rng = np.random.default_rng(1)
        octx = orc_mod.OracleContext(LOGN, prm.moduli)
        all_idx = prm.q_idx + prm.p_idx

        def rl(idx):
            return np.stack([rng.integers(0, prm.moduli[p], size=N, dtype=np.uint64) for p in idx])
        a0, a1, b0, b1 = rl(prm.q_idx), rl(prm.q_idx), rl(prm.q_idx), rl(prm.q_idx)
        evk = np.stack([np.stack([rl(all_idx) for _ in range(2)]) for _ in range(prm.dnum)])
        t0 = time.perf_counter()
        octx.hmult_relin(orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF, True, prm.q_idx, prm.p_idx, prm.dnum, a0, a1, b0, b1, evk)
        dt = time.perf_counter() - t0
        return 1.0 / dt, "1 HMult+relin+rescale (L=24, K=1, dnum=24), oracle port with OpenMP over limbs"


class NttWorkload(Workload):
    name = "ntt_fwd_inv_N65536_48limbs_x8_u64"
    metric = "ntt_limb_transforms_per_s"
    unit = "limb-NTT/s"

    def __init__(self):
        self.moduli = params.config_ntt(LOGN, 48)
        self.idx = [l for _ in range(8) for l in range(48)]
        self.ops_per_step = 2 * len(self.idx)  # forward + inverse

    def setup(self, lib, torch, rank, world=1, sharded=False):
        from cerium_b200 import _capi
        self.torch = torch
        self.ctx = _capi.Context(lib, self.moduli, 64, device=torch.cuda.current_device())
        gen = torch.Generator(device="cuda").manual_seed(0xCE210002 + rank)
        self.x = _rand_limbs_gpu(torch, self.moduli, self.idx, (), gen)
        self.y = torch.empty_like(self.x)
        self.alg_bytes = 2 * 2 * len(self.idx) * N * 8
        self.host_in = torch.empty(self.x.shape, dtype=torch.int64).pin_memory()
        self.host_in.copy_(self.x.cpu())
        self.host_out = torch.empty(self.x.shape, dtype=torch.int64).pin_memory()
        self.gpu_launches_per_step = 4

    def step(self):
        s = self.torch.cuda.current_stream().cuda_stream
        self.ctx.ntt_forward(self.y.data_ptr(), self.x.data_ptr(), self.idx, stream=s)
        self.ctx.ntt_inverse(self.y.data_ptr(), self.y.data_ptr(), self.idx, stream=s)

    def verify(self, orc_mod):
        """Forward transform of every limb against the oracle, then the round trip on the device."""
        torch = self.torch
        s = torch.cuda.current_stream().cuda_stream
        self.ctx.ntt_forward(self.y.data_ptr(), self.x.data_ptr(), self.idx, stream=s)
        torch.cuda.synchronize()
        octx = orc_mod.OracleContext(LOGN, self.moduli)
        want = octx.ntt_forward(self.x.cpu().numpy().view(np.uint64), self.idx)
        ok = bool(np.array_equal(self.y.cpu().numpy().view(np.uint64), want))
        self.ctx.ntt_inverse(self.y.data_ptr(), self.y.data_ptr(), self.idx, stream=s)
        torch.cuda.synchronize()
        return ok and bool(torch.equal(self.y, self.x))

    def e2e_step(self):
        if getattr(self, "pipe", None) is None:
            from cerium_b200.host_pipeline import HostPipeline

            def op(ins, outs, stream):
                self.ctx.ntt_forward(outs[0].data_ptr(), ins[0].data_ptr(), self.idx, stream=stream)
                self.ctx.ntt_inverse(outs[0].data_ptr(), outs[0].data_ptr(), self.idx, stream=stream)
            self.pipe = HostPipeline(self.torch, [self.x.shape], [self.x.shape], op)
        self.pipe.submit([self.host_in])
        return self.pipe.in_bytes, self.pipe.out_bytes

    def roofline_setup(self):
        self.rl_bytes = 2 * len(self.idx) * N * 8
        self.rl_name = "forward NTT (column pass + row pass), %d limbs u64" % len(self.idx)

    def roofline_step(self):
        self.ctx.ntt_forward(self.y.data_ptr(), self.x.data_ptr(), self.idx,
                             stream=self.torch.cuda.current_stream().cuda_stream)

    def cpu_sample(self, orc_mod):
        rng = np.random.default_rng(1)
        octx = orc_mod.OracleContext(LOGN, self.moduli)
        x = np.stack([rng.integers(0, self.moduli[p], size=N, dtype=np.uint64) for p in self.idx])
        t0 = time.perf_counter()
        f = octx.ntt_forward(x, self.idx)
        octx.ntt_inverse(f, self.idx)
        dt = time.perf_counter() - t0
        return self.ops_per_step / dt, "forward+inverse NTT of 384 limbs, oracle port (Harvey lazy butterflies), OpenMP over limbs"


class HoistedWorkload(HRotWorkload):
    """Eight rotations of one ciphertext that share the ModUp (hoisting, the baby steps of a BSGS
    matrix-vector product: cerium/compiler/backend/compiler.cc:958-1153): one cerium_hoisted_begin,
    then per rotation inner product + ModDown + automorphism with a pre-permuted key."""
    name = "hoisted_8_rotations_N65536_L35_K5_dnum7_u64"
    metric = "hoisted_rotations_per_s"
    unit = "rotations/s"
    ops_per_step = 8

    def setup(self, lib, torch, rank, world=1, sharded=False):
        super().setup(lib, torch, rank, world, False)
        prm = self.prm
        gen = torch.Generator(device="cuda").manual_seed(0xCE210013 + rank)
        all_idx = prm.q_idx + prm.p_idx
        self.evks = [self.evk] + [_rand_limbs_gpu(torch, prm.moduli, all_idx, (prm.dnum, 2), gen)
                                  for _ in range(self.ops_per_step - 1)]
        self.elts = [lib.galois_elt_from_step(1 << k, LOGN) for k in range(self.ops_per_step)]
        self.houts = [torch.empty_like(self.cts[0]) for _ in range(self.ops_per_step)]
        self.alg_bytes = (2 * prm.L + self.ops_per_step * (prm.dnum * 2 * (prm.L + prm.K) + 2 * prm.L)) * N * 8
        # begin: iNTT pair, BConv, NTT pair; per rotation: inner product, iNTT pair, BConv, SuD pair (the automorphism is the SuD tail's store pattern)
        self.gpu_launches_per_step = 5 + self.ops_per_step * 6

    def _run(self, ct, outs, stream):
        self.ks.hoisted_begin(ct[1].data_ptr(), stream)
        for k in range(self.ops_per_step):
            o = outs[k]
            self.ks.hoisted_rotate(o[0].data_ptr(), o[1].data_ptr(), ct[0].data_ptr(), ct[1].data_ptr(),
                                   self.evks[k].data_ptr(), self.elts[k], stream)

    def step(self):
        k = self.i % self.n_cts
        self.i += 1
        self._run(self.cts[k], self.houts, self.torch.cuda.current_stream().cuda_stream)

    def e2e_step(self):
        if getattr(self, "pipe", None) is None:
            from cerium_b200.host_pipeline import HostPipeline

            def op(ins, outs, stream):
                self._run(ins[0], outs, stream)
            self.pipe = HostPipeline(self.torch, [self.cts[0].shape], [self.cts[0].shape] * self.ops_per_step, op)
        self.pipe.submit([self.host_ins[0]])
        return self.pipe.in_bytes, self.pipe.out_bytes

    def cpu_sample(self, orc_mod):
        v, sample = super().cpu_sample(orc_mod)
        return v, sample + " (one plain rotation; the CPU port does not hoist)"


class BsgsWorkload(HRotWorkload):
    """One BSGS multiply-accumulate with 8 baby x 8 giant steps (64 diagonals) on the HRot parameter
    set: the linear-transform stage of bootstrapping (CoeffToSlot / SlotToCoeff,
    cerium/compiler/backend/compiler.cc:2457-2822) through cerium_bsgs_apply: 7 hoisted baby
    rotations, the plaintext multiply-accumulate of all giant steps in two passes over the rotated
    copies, 7 giant-step key switches accumulated in the extended basis, one ModDown."""
    name = "bsgs_8x8_N65536_L35_K5_dnum7_u64"
    metric = "bsgs_linear_transforms_per_s"
    unit = "transforms/s"
    ops_per_step = 1
    G = 8

    def setup(self, lib, torch, rank, world=1, sharded=False):
        super().setup(lib, torch, rank, world, False)
        from cerium_b200.bsgs import BsgsMultiplyAccumulate
        prm, G = self.prm, self.G
        gen = torch.Generator(device="cuda").manual_seed(0xCE210023 + rank)
        all_idx = prm.q_idx + prm.p_idx
        key = lambda: _rand_limbs_gpu(torch, prm.moduli, all_idx, (prm.dnum, 2), gen)  # noqa: E731
        self.baby_keys = [key() for _ in range(G - 1)]
        self.giant_keys = [key() for _ in range(G - 1)]
        self.baby_elts = [lib.galois_elt_from_step(i, LOGN) for i in range(1, G)]
        self.giant_elts = [lib.galois_elt_from_step(G * j, LOGN) for j in range(1, G)]
        self.pts = [[_rand_limbs_gpu(torch, prm.moduli, prm.q_idx, (), gen) for _ in range(G)] for _ in range(G)]
        self.op = BsgsMultiplyAccumulate(self.ctx, self.ks, G, G,
                                         lambda shape: torch.empty(tuple(shape), dtype=torch.int64, device="cuda"),
                                         lambda t: t.data_ptr())
        self.bout = torch.empty_like(self.cts[0])
        limb = N * 8
        # ciphertext in and out, 14 keys, 64 plaintexts
        self.alg_bytes = (4 * prm.L + 2 * (G - 1) * prm.dnum * 2 * (prm.L + prm.K) + G * G * prm.L) * limb
        # hoisted begin 5, baby rotation 6 each, 2 plaintext passes, 2 rotation sums, per giant step
        # iNTT pair + BConv + NTT pair + inner product, final ModDown 5
        self.gpu_launches_per_step = 5 + (G - 1) * 6 + 2 + 2 + (G - 1) * 6 + 5

    def _run(self, ct, out, stream):
        self.op.run(out, ct, self.pts, self.baby_keys, self.giant_keys, self.baby_elts, self.giant_elts, stream)

    def step(self):
        k = self.i % self.n_cts
        self.i += 1
        self._run(self.cts[k], self.bout, self.torch.cuda.current_stream().cuda_stream)

    def verify(self, orc_mod):
        """The whole transform against the oracle's restatement of the reference lowering (baby steps
        as hoisted rotations, extended-basis accumulation, one ModDown)."""
        torch, prm, G = self.torch, self.prm, self.G
        u = lambda t: t.cpu().numpy().view(np.uint64)  # noqa: E731
        ct = self.cts[0]
        self._run(ct, self.bout, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        octx = orc_mod.OracleContext(LOGN, prm.moduli)
        c0, c1 = u(ct[0]), u(ct[1])
        baby = [np.stack([c0, c1])]
        for j in range(1, G):
            k0, k1 = octx.keyswitch(orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, c1,
                                    u(self.baby_keys[j - 1]))
            k0 = np.stack([orc_mod.ew("add", prm.moduli[p], k0[i], c0[i]) for i, p in enumerate(prm.q_idx)])
            e = self.baby_elts[j - 1]
            baby.append(np.stack([np.stack([orc_mod.apply_galois_ntt(e, LOGN, k[i]) for i in range(prm.L)]) for k in (k0, k1)]))
        pts = np.stack([np.stack([u(t) for t in row]) for row in self.pts])
        keys = np.stack([np.zeros_like(u(self.giant_keys[0]))] + [u(k) for k in self.giant_keys])
        w0, w1 = octx.bsgs(orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF, prm.q_idx, prm.p_idx, prm.dnum, 0, np.stack(baby), pts,
                           np.ones((G, G), dtype=np.uint8), [1] + list(self.giant_elts), keys)
        got = u(self.bout)
        return bool(np.array_equal(got[0], w0) and np.array_equal(got[1], w1))

    def e2e_step(self):
        if getattr(self, "pipe", None) is None:
            from cerium_b200.host_pipeline import HostPipeline

            def op(ins, outs, stream):
                self._run(ins[0], outs[0], stream)
            self.pipe = HostPipeline(self.torch, [self.cts[0].shape], [self.cts[0].shape], op)
        self.pipe.submit([self.host_ins[0]])
        return self.pipe.in_bytes, self.pipe.out_bytes

    def cpu_sample(self, orc_mod):
        v, sample = super().cpu_sample(orc_mod)
        # 14 key switches dominate one transform on the CPU as well
        return v / (2 * (self.G - 1)), sample + " (one rotation timed; a transform is counted as its 14 rotations)"


class BootstrapWorkload(Workload):
    """One CKKS bootstrap as the operator list of cerium_b200/bootstrap.py (the structure of the reference's
    benchmarks/bootstrap_32K/bootstrap.py:299-358 for the parameterisation the benchmark names): ModRaise of
    a two-limb ciphertext to 34 limbs, CoeffToSlot as three 8 x 8 BSGS multiply-accumulates with the rescale
    folded in, conjugation split, a degree-63 Chebyshev polynomial (16 HMults) and two double-angle steps on
    both parts, SlotToCoeff as three more BSGS stages: 15 levels, 103 key switches.  Keys, diagonals and
    coefficients are seeded uniform residues of the real shapes (30 GB on the device)."""
    name = "bootstrap_N65536_top34_K5_dnum7_c2s3_s2c3_cheb63_da2_u64"
    metric = "bootstrap_latency_ms"
    unit = "ms"
    ops_per_step = 1
    latency_metric = True

    def __init__(self):
        self.prm = params.config_hrot(LOGN, 35, 5, 7)

    def _make(self, tag, lead, idx):
        import zlib
        gen = self.torch.Generator(device="cuda").manual_seed(zlib.crc32(repr(tag).encode()))
        return _rand_limbs_gpu(self.torch, self.prm.moduli, list(idx), tuple(lead), gen)

    def setup(self, lib, torch, rank, world=1, sharded=False):
        from cerium_b200 import _capi, bootstrap as bs
        self.torch, self.bs, self.lib = torch, bs, lib
        prm = self.prm
        self.ctx = _capi.Context(lib, prm.moduli, 64, device=torch.cuda.current_device())
        self.shape = bs.BootstrapShape(top=prm.L - 1)
        self.material = bs.BootstrapMaterial(prm.moduli, prm.q_idx, prm.p_idx, prm.dnum, self.shape, self._make,
                                             lambda step: lib.galois_elt_from_step(step, LOGN))
        self.ev = bs.GpuEvaluator(torch, _capi, self.ctx, self.material, _capi.BCONV_EXACT, _capi.ROUND_HALF)
        gen = torch.Generator(device="cuda").manual_seed(0xCE210004 + rank)
        self.ct2 = [_rand_limbs_gpu(torch, prm.moduli, prm.q_idx[:2], (), gen) for _ in range(2)]
        self.host_in = torch.stack(self.ct2).cpu().pin_memory()
        out_level = self.shape.top - self.shape.levels_used
        self.out_shape = (2, out_level, N)
        # the first run creates the plans, keys and diagonals of every level
        self.step()
        torch.cuda.synchronize()
        n = self.ev.count.n
        self.op_counts = dict(n)
        # launches: ModRaise 19; a BSGS stage 5 + 7 * 6 + 2 + 2 + 8 * 6 + 5; an HMult 15; a conjugation 11;
        # a rescale 4; every other pass 1
        self.gpu_launches_per_step = (19 * n["mod_raise"] + 104 * n["bsgs"] + 15 * n["hmult"] + 11 + 4 * n["rescale"]
                                      + n["ewise"] + 2 * n["pt_mac"])
        self.ev.count.n = {}
        self.alg_bytes = 0

    def step(self):
        self.ev.stream = self.torch.cuda.current_stream().cuda_stream
        self.result = self.bs.bootstrap(self.ev, self.shape, self.ct2)

    def verify(self, orc_mod):
        """ModRaise and the first CoeffToSlot stage at full size against the oracle (15 key switches of 34
        limbs, the plaintext products, one ModDown with the rescale folded in); the whole operator list is
        compared with the oracle at a reduced shape by tests/test_gpu_bootstrap.py."""
        from tests.bootstrap_checker import OracleEvaluator
        torch, m = self.torch, self.material
        u = lambda t: t.cpu().numpy().view(np.uint64)  # noqa: E731

        class HostMaterial:
            """The device material seen from the host: the same buffers, copied on first use."""
            def __init__(self, dev):
                self.d = dev
                self.moduli, self.q_idx, self.p_idx, self.top = dev.moduli, dev.q_idx, dev.p_idx, dev.top
                self.lift_key = u(dev.lift_key)
                self.dnum_at = dev.dnum_at

            def stage(self, stage, level):
                st = self.d.stage(stage, level)
                h = lambda t: None if t is None else u(t)  # noqa: E731
                return type(st)(st.g, st.n_giant, [h(t) for t in st.pts], [h(t) for t in st.baby_keys], st.baby_elts,
                                [h(t) for t in st.giant_keys], st.giant_elts)
        oe = OracleEvaluator(HostMaterial(m), orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF)
        self.ev.stream = torch.cuda.current_stream().cuda_stream
        g = self.ev.bsgs(self.ev.mod_raise(self.ct2), ("c2s", 0))
        torch.cuda.synchronize()
        w = oe.bsgs(oe.mod_raise([u(self.ct2[0]), u(self.ct2[1])]), ("c2s", 0))
        self.ev.count.n = {}
        return bool(np.array_equal(u(g.c0[:g.level]), w.c0) and np.array_equal(u(g.c1[:g.level]), w.c1))

    def e2e_step(self):
        if getattr(self, "pipe", None) is None:
            from cerium_b200.host_pipeline import HostPipeline

            def op(ins, outs, stream):
                self.ev.stream = stream
                r = self.bs.bootstrap(self.ev, self.shape, [ins[0][0], ins[0][1]])
                outs[0][0].copy_(r.c0[:r.level], non_blocking=True)
                outs[0][1].copy_(r.c1[:r.level], non_blocking=True)
            self.pipe = HostPipeline(self.torch, [self.host_in.shape], [self.out_shape], op)
        self.pipe.submit([self.host_in])
        return self.pipe.in_bytes, self.pipe.out_bytes

    def roofline_setup(self):
        HRotWorkload.roofline_setup(self)

    def roofline_step(self):
        HRotWorkload.roofline_step(self)

    def cpu_sample(self, orc_mod):
        """One key switch of 34 limbs on the CPU port, scaled by the bootstrap's 103 key switches (they are
        nine tenths of its time on the GPU as well)."""
        prm = self.prm
        rng = np.random.default_rng(1)
        octx = orc_mod.OracleContext(LOGN, prm.moduli)
        q_idx = prm.q_idx[:34]
        all_idx = q_idx + prm.p_idx
        rl = lambda idx: np.stack([rng.integers(0, prm.moduli[p], size=N, dtype=np.uint64) for p in idx])  # noqa: E731
        c = rl(q_idx)
        evk = np.stack([np.stack([rl(all_idx) for _ in range(2)]) for _ in range(7)])
        t0 = time.perf_counter()
        octx.keyswitch(orc_mod.BCONV_EXACT, orc_mod.ROUND_HALF, q_idx, prm.p_idx, 7, c, evk)
        dt = time.perf_counter() - t0
        return 103 * dt * 1e3, "one key switch (L=34, K=5, dnum=7) on the oracle port x the 103 key switches of a bootstrap"


class _DevicePtr:
    """A raw device limb as something torch can wrap without a copy."""
    def __init__(self, ptr, words):
        self.__cuda_array_interface__ = {"shape": (words,), "typestr": "<i4", "data": (int(ptr), False), "version": 2}


class BootstrapProgramWorkload(Workload):
    """The reference's OWN bootstrapping benchmark (benchmarks/bootstrap_32K/bootstrap.py: 2^15 slots, 33 levels,
    28-bit primes, sparse-secret encapsulation; one GPU: 462 records, 195 key digits, 259 plaintexts), compiled by
    the reference's compiler (tests/golden/programs/make_programs.py) and replayed by this library's executor
    through the Python surface of cerium_b200/runtime.py - the sequence of benchmarks/bootstrap_32K/
    bootstrap_runner.py:83-170.  The transform, base-conversion and SuD records run on this library's kernels; the
    element-wise records run on the kernels the compiler generated for the program (the plugin contract).  With
    --gpus N the build of the program for N GPUs runs as N processes, its drm / ags / ard records on NCCL.
    Keys are generated here from a seeded secret; plaintext diagonals and coefficients are the benchmark's own
    values.  `verified` = the bootstrapped ciphertext decrypts to its input slots with at least 15 bits."""
    name = "reference_bootstrap_32K_33levels_compiled_program_u32"
    metric = "bootstrap_latency_ms"
    unit = "ms"
    ops_per_step = 1
    latency_metric = True
    dtype = "u32"
    inflight = 1

    def setup(self, lib, torch, rank, world=1, sharded=False, comm=None, **_):
        import lzma
        import random
        import shutil
        import tempfile
        from cerium_b200 import _capi, runtime
        self.torch, self.rank, self.world, self.comm = torch, rank, world, comm
        root = os.path.dirname(os.path.abspath(__file__))
        tag, fn = "bootstrap_32K_%dgpu" % world, "bootstrap_32Kslots_33levels_%dgpus" % world
        fixtures = os.path.join(root, "tests", "golden", "programs", tag)
        built = os.path.join(root, "oracle", "_ref", "programs", tag)
        need = [os.path.join(built, "raw_inputs.npz")] + [os.path.join(built, "function_map_%d.orig.so" % p) for p in range(world)]
        if not os.path.isdir(fixtures) or not all(os.path.exists(f) for f in need):
            raise SystemExit("bench.py: the compiled bootstrapping program for %d GPU(s) is not built "
                             "(python tests/golden/programs/make_programs.py)" % world)
        self.tmp = tempfile.mkdtemp(prefix="cerium_boot_r%d_" % rank)
        d = os.path.join(self.tmp, fn)
        os.makedirs(d)
        for f in ["program_inputs"] + ["%s%d" % (k, p) for p in range(world) for k in ("functions", "inputs")]:
            with lzma.open(os.path.join(fixtures, f + ".xz"), "rb") as src, open(os.path.join(d, f), "wb") as dst:
                dst.write(src.read())
        for p in range(world):
            shutil.copy(os.path.join(built, "function_map_%d.orig.so" % p), os.path.join(d, "function_map_%d.so" % p))
        z = np.load(os.path.join(built, "raw_inputs.npz"))
        raw = {k[2:]: (z[k][()] if z[k].ndim == 0 else z[k], float(z["s:" + k[2:]])) for k in z.files if k.startswith("v:")}
        slots = N // 2
        primes = params.reference_primes_28bit(64, LOGN)
        rnd = random.Random(10)

        def secret(weight):
            key = [0] * N
            for pos in rnd.sample(range(N), weight):
                key[pos] = rnd.choice((-1, 1))
            return key
        self.context = runtime.Context(slots, primes, lib=lib, device=torch.cuda.current_device())
        seed = np.random.default_rng(10).integers(0, 2 ** 32 - 1, size=8).tolist()
        self.ectx = runtime.CKKSEncryptorContext(self.context, secret(slots), secret(32), seed)
        self.encryptor = runtime.CKKSEncryptor(self.ectx, seed)
        self.scale = primes[1] * primes[0] / (1 << 5)
        self.slots_in = np.exp(1j * np.random.default_rng(10).uniform(0, 2 * np.pi, slots))
        prog = runtime.FusedKernelProgram(self.context, self.tmp, fn)
        self.fn = prog.make_program(world, {}, runtime.RawInputsWrapper(raw), partition=rank, comm=comm,
                                    encryptor_context=self.ectx)[fn]
        gen = runtime.IOGenerator(self.context)
        self.ct_in = gen.generate_ciphertext_inputs(os.path.join(d, "program_inputs"),
                                                    runtime.RawInputsWrapper({"x": (self.slots_in, self.scale)}), self.ectx)
        self.fn.copy_ciphertext_inputs_to_gpu("", world, self.ct_in)
        self.program = self.fn.program
        recs = _capi.inspect_program(lib, os.path.join(d, "functions%d" % rank))
        self.gpu_launches_per_step = self.program.num_steps
        self.transform_limbs = sum(r["outputs"] for r in recs if r["type"] in ("ntt", "int"))
        self.ntt_limbs = max(r["outputs"] for r in recs if r["type"] == "ntt")
        # algorithmic bytes of a run: every record reads its inputs and writes its outputs once
        self.alg_bytes = sum((r["outputs"] + r["inputs"]) * N * 4 for r in recs if r["type"] != "mov")
        # the limbs of the input and output terms this partition holds, as torch views of program memory
        def views(stream_name):
            out = []
            for term, desc, bases in self.fn.streams.get(stream_name, []):
                for l in self.fn._mine(term, bases):
                    t = torch.as_tensor(_DevicePtr(self.program.memory("%s(%d)" % (term, l)), N), device="cuda")
                    out.append((desc, l, t))
            return out
        self.in_views, self.out_views = views("Ciphertext Stream"), views("Output Stream")

    def step(self):
        self.program.run(self.torch.cuda.current_stream().cuda_stream)
        self.queued = getattr(self, "queued", 0) + 1
        if self.world > 1 and self.queued % 8 == 0:
            # a run holds tens of exchange records on up to three communicators: the host stays at most eight
            # runs ahead of the GPUs (a run takes milliseconds, the wait is not seen in the timing)
            self.torch.cuda.current_stream().synchronize()

    def verify(self, orc_mod):
        import torch.distributed as dist
        del orc_mod                                  # checked by decryption, not by the CPU restatement
        self.step()
        self.torch.cuda.synchronize()
        ct = self.fn.get_program_outputs()["z"]
        if self.world > 1:
            from cerium_b200 import runtime
            parts = [None] * self.world
            dist.all_gather_object(parts, (ct.rns_base_ids, ct.c0, ct.c1))
            ids = sorted(i for p in parts for i in p[0])
            r0 = {i: p[1][k] for p in parts for k, i in enumerate(p[0])}
            r1 = {i: p[2][k] for p in parts for k, i in enumerate(p[0])}
            ct = runtime.Ciphertext(np.stack([r0[i] for i in ids]), np.stack([r1[i] for i in ids]), ids)
        z = np.asarray(self.encryptor.decrypt_and_decode(ct, self.scale))
        self.precision_bits = float(-np.log2(np.max(np.abs(z - self.slots_in))))
        return bool(self.precision_bits > 15)

    def e2e_step(self):
        if getattr(self, "pipe", None) is None:
            from cerium_b200.host_pipeline import HostPipeline
            torch = self.torch

            def op(ins, outs, stream):
                for k, (_, _, view) in enumerate(self.in_views):
                    view.copy_(ins[0][k], non_blocking=True)
                self.program.run(stream)
                for k, (_, _, view) in enumerate(self.out_views):
                    outs[0][k].copy_(view, non_blocking=True)
            self.pipe = HostPipeline(torch, [(len(self.in_views), N)], [(len(self.out_views), N)], op, dtype=torch.int32)
            rows = []
            for desc, l, _ in self.in_views:
                var, poly = desc.split(":")
                ct = self.ct_in[var]
                rows.append((ct.c0 if poly == "c0" else ct.c1)[ct.rns_base_ids.index(l)])
            # a partition of a build for many GPUs may hold none of the (two-limb) input ciphertext
            stacked = np.stack(rows).view(np.int32).copy() if rows else np.zeros((0, N), dtype=np.int32)
            self.host_in = torch.from_numpy(stacked).pin_memory()
        self.pipe.submit([self.host_in])
        return self.pipe.in_bytes, self.pipe.out_bytes

    def roofline_setup(self):
        self.rl_idx = list(range(min(self.ntt_limbs, 64)))
        gen = self.torch.Generator(device="cuda").manual_seed(5)
        self.rl_buf = self.torch.randint(0, 1 << 27, (len(self.rl_idx), N), dtype=self.torch.int32, device="cuda", generator=gen)
        self.rl_bytes = 2 * len(self.rl_idx) * N * 4
        self.rl_name = "forward NTT (column pass + row pass), %d limbs u32 (the program's widest ntt record)" % len(self.rl_idx)

    def roofline_step(self):
        self.context.handle.ntt_forward(self.rl_buf.data_ptr(), self.rl_buf.data_ptr(), self.rl_idx,
                                        stream=self.torch.cuda.current_stream().cuda_stream)

    def cpu_sample(self, orc_mod):
        """The transforms of one run on the CPU port (a lower bound of the CPU time: element-wise products, base
        conversions and divisions are left out)."""
        rng = np.random.default_rng(1)
        primes = params.reference_primes_28bit(64, LOGN)
        octx = orc_mod.OracleContext(LOGN, primes)
        idx = list(range(48))
        x = np.stack([rng.integers(0, primes[p], size=N, dtype=np.uint64) for p in idx])
        t0 = time.perf_counter()
        octx.ntt_forward(x, idx)
        dt = time.perf_counter() - t0
        limbs = getattr(self, "transform_limbs", 9698)   # the one-GPU build when no program is loaded (reference arm)
        return dt / len(idx) * limbs * 1e3, ("48 forward NTTs on the oracle port, scaled to the %d limb transforms of one run; "
                                             "lower bound, the other records are left out" % limbs)


WORKLOADS = {"hrot": HRotWorkload, "hmult": HMultWorkload, "ntt": NttWorkload, "hoisted": HoistedWorkload,
             "bsgs": BsgsWorkload, "bootstrap": BootstrapWorkload, "bootstrap_program": BootstrapProgramWorkload}


# ---------------------------------------------------------------------------------------

def run_reference_arm(args, wl):
    """The reference's own CPU implementation of the path cannot be built here (it needs Microsoft
    SEAL 4.1.1, absent), so this arm times the oracle port of the same algorithm on the host cores."""
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    import oracle
    # all the host threads there are, also under torchrun (which exports OMP_NUM_THREADS=1)
    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    vals = []
    sample = ""
    for _ in range(max(1, min(args.warmup, 1))):
        wl.cpu_sample(oracle)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        v, sample = wl.cpu_sample(oracle)
        vals.append(v)
    wall = time.perf_counter() - t0
    value = float(np.mean(vals))
    ops = getattr(wl, "ops_per_step", 1)
    line = {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": value if getattr(wl, "latency_metric", False) else 1e3 * ops / value,
        "higher_is_better": not getattr(wl, "latency_metric", False), "scaling": "weak", "vs_baseline": None,
        "dtype": getattr(wl, "dtype", "u64"), "data": "synthetic",
        "config": {"workload": wl.name},
        "note": "CPU port of the reference algorithm (SEAL-based reference runtime not buildable here)",
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
                         "port_quality": PORT_QUALITY, "sample": sample},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": wall,
    }
    print(json.dumps(line), flush=True)


def bind_to_gpu_numa(torch, local_rank):
    """Best effort: run this process (and so first-touch its pinned buffers) on the NUMA node of its GPU."""
    try:
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev = torch.cuda.get_device_properties(local_rank).pci_device_id
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/numa_node" % (dom, bus, dev)
        node = int(open(path).read().strip())
        if node < 0:
            return None
        cpus = []
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.extend(range(int(lo), int(hi or lo) + 1))
        allowed = sorted(set(cpus) & os.sched_getaffinity(0))
        if allowed:
            os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def time_blocks(torch, dist, world, wl, steps, blocks, barrier):
    """`blocks` timed regions of `steps` steps each (CUDA events on the current stream, side streams
    forked and joined inside, max over ranks); returns the list of milliseconds."""
    out = []
    for _ in range(blocks):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        wl.fork()
        for _ in range(steps):
            wl.step()
        wl.join()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out.append(ms)
    return out


def roofline_of(torch, wl, peak, peak_kind, iters=20):
    wl.roofline_setup()
    for _ in range(3):
        wl.roofline_step()
    torch.cuda.synchronize()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for _ in range(iters):
        wl.roofline_step()
    r1.record()
    torch.cuda.synchronize()
    rl_ms = r0.elapsed_time(r1) / iters
    achieved = wl.rl_bytes / (rl_ms / 1e3) / 1e9
    u32 = getattr(wl, "dtype", "u64") == "u32"
    limbs = wl.rl_bytes // (2 * N * (4 if u32 else 8))
    return {"bound": "hbm", "kernel": wl.rl_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "traffic": None if u32 else NTT_PAIR_DRAM_BYTES_PER_LIMB * limbs,
            "traffic_source": ("no ncu capture of the 32-bit transform pair" if u32 else
                               "profiles/ (ncu capture of the forward NTT pair, scaled by limbs)"),
            "peak_kind": peak_kind, "ms_per_launch_pair": rl_ms, "algorithmic_bytes": wl.rl_bytes}, rl_ms, limbs


def sub_measurement(torch, lib, name, steps, peak, peak_kind, verify_with):
    """A short run of another workload (its own inputs, verification, timing and roofline) for the default line."""
    wl = WORKLOADS[name]()
    wl.setup(lib, torch, 0, 1, False)
    verified = wl.verify(verify_with) if verify_with is not None else None
    if verified is False:
        return {"workload": wl.name, "verified": False}
    for _ in range(10):
        wl.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        wl.step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    rl, _, _ = roofline_of(torch, wl, peak, peak_kind, iters=10)
    out = {"workload": wl.name, "metric": wl.metric, "value": wl.ops_per_step / (ms / 1e3), "unit": wl.unit,
           "ms_per_step": ms, "steps": steps, "verified": verified, "roofline": rl,
           "step_algorithmic_gbs": wl.alg_bytes / (ms / 1e3) / 1e9}
    del wl
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="hrot")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle comparison before timing")
    ap.add_argument("--no-sub", action="store_true", help="skip the short hmult / ntt measurements of the default line")
    ap.add_argument("--blocks", type=int, default=5, help="timed blocks of --steps steps (the first is the headline)")
    ap.add_argument("--parallelism", choices=["auto", "limb", "replica"], default="auto",
                    help="N > 1, hrot: 'limb' (what 'auto' picks) shards every ciphertext and key by RNS limb over the "
                         "ranks, NCCL all-gathers where limbs must meet, several operations in flight; 'replica' runs "
                         "independent ciphertexts per rank with no collective")
    ap.add_argument("--inflight", type=int, default=None,
                    help="independent operations in flight per rank, each on its own plan and stream (hrot; default 2 "
                         "on one GPU, 4 limb-sharded)")
    ap.add_argument("--ext", choices=["split", "replicated"], default="split",
                    help="limb-sharded: extension limbs split over the ranks, or replicated on every rank")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]()
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 3
        args.warmup = args.warmup if args.warmup is not None else 1
        run_reference_arm(args, wl)
        return
    slow = args.workload in ("bootstrap", "bsgs", "bootstrap_program")
    args.steps = args.steps if args.steps is not None else (20 if args.workload == "bootstrap" else 50 if args.workload == "bootstrap_program" else 200 if slow else 2000)
    args.warmup = max(3, args.warmup if args.warmup is not None else (3 if slow else 50))

    # a stage that stops making progress (a collective whose peers never arrive) ends the run instead of waiting for
    # the caller's limit; CERIUM_BENCH_WATCHDOG_S=0 switches it off
    dog = Watchdog(float(os.environ.get("CERIUM_BENCH_WATCHDOG_S", "600")))
    if args.workload == "bootstrap_program" and env_int("WORLD_SIZE", 1) > 1:
        # the configuration tests/test_runtime_facade.py runs the program's builds for 2 and 4 GPUs in: groups of
        # neighbouring ranks get communicators of their own, and NVLink multicast stays out of it
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

    import torch
    import torch.distributed as dist
    from cerium_b200 import _capi

    world = env_int("WORLD_SIZE", 1)
    rank = env_int("RANK", 0)
    local_rank = env_int("LOCAL_RANK", 0)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    numa = bind_to_gpu_numa(torch, local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = _capi.load()
    dog.at("setup")
    sharded = world > 1 and ((args.parallelism in ("auto", "limb") and args.workload == "hrot") or args.workload == "bootstrap_program")
    comm = None
    if sharded and args.workload == "bootstrap_program":
        from cerium_b200 import sharded as sh
        comm = sh.nccl_comm(lib, rank, world, local_rank)
        wl.setup(lib, torch, rank, world, True, comm=comm)
    elif sharded:
        from cerium_b200 import sharded as sh
        comm = sh.nccl_comm(lib, rank, world, local_rank)
        wl.setup(lib, torch, rank, world, True, comm=comm, ext_split=args.ext == "split",
                 inflight=max(1, args.inflight if args.inflight is not None else 4))
    else:
        if args.workload == "hrot":
            # replicas (N > 1, --parallelism replica) run one operation at a time; one GPU runs two
            wl.setup(lib, torch, rank, world, False,
                     inflight=max(1, args.inflight if args.inflight is not None else (2 if world == 1 else 1)))
        else:
            wl.setup(lib, torch, rank, world, False)
    ops = wl.ops_per_step
    job_ops = 1 if sharded else world   # ops per step of the whole job: one sharded op, or one per replica

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # parity first: one operation on the benchmark's own inputs against the oracle (the checker; sharded:
    # against the one-GPU operation the oracle pins), outside every timed region; no value is printed for
    # a path whose result is wrong
    verified = None
    oracle = None
    dog.at("verify")
    if not args.no_verify:
        import oracle
        oracle.set_num_threads(max(1, len(os.sched_getaffinity(0)) // max(1, world)))
        verified = wl.verify(oracle)
        if world > 1 and verified is not None:
            t = torch.tensor([1 if verified else 0], dtype=torch.int32, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            verified = bool(t.item())
        if verified is False:
            raise SystemExit("bench.py: %s does not match the oracle on the benchmark inputs; nothing is timed" % wl.name)

    dog.at("warm-up")
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    wl.fork()
    for _ in range(args.warmup):
        wl.step()
    wl.join()
    barrier()
    sampler.mark_start()
    # under a profiler started with its collection off, only the timed blocks are collected
    profile_range = bool(os.environ.get("CERIUM_BENCH_PROFILE_RANGE"))
    if profile_range:
        torch.cuda.profiler.start()
    dog.at("timed blocks")
    block_ms = time_blocks(torch, dist, world, wl, args.steps, max(1, args.blocks), barrier)
    if profile_range:
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    ms = block_ms[0]

    clocks = sampler.stop() if rank == 0 else None     # the clock record covers the timed blocks only
    dog.at("roofline kernel and probe")
    peak, peak_kind = measured_peaks()
    # the roofline kernel is timed alone against the burst copy rate: give the GPU a moment off the timed loop's
    # power cap first, so that the kernel is not measured at the loop's lowered clock
    torch.cuda.synchronize()
    time.sleep(1.5)
    roofline, rl_ms, rl_limbs = roofline_of(torch, wl, peak, peak_kind)
    probe = probe_int_pipe(local_rank) if rank == 0 else None

    # latency of ONE operation (nothing else in flight) beside the throughput of several
    dog.at("side measurements")
    side = {}
    if getattr(wl, "inflight", 1) > 1 and args.workload == "hrot":
        keep = wl.inflight
        wl.inflight = 1
        lsteps = max(5, min(args.steps, 200))
        side["latency_ms_one_op_in_flight"] = time_blocks(torch, dist, world, wl, lsteps, 1, barrier)[0] / lsteps
        wl.inflight = keep
    # N > 1: the other parallelism beside the headline, and the collectives of one sharded operation alone
    if sharded and args.workload == "hrot":
        for _ in range(5):
            wl.collective_step()
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(50):
            wl.collective_step()
        c1.record()
        barrier()
        t = torch.tensor([c0.elapsed_time(c1) / 50], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        side["collective_ms_per_op"] = float(t.item())
        # replicas: independent ciphertexts per GPU, no collective (weak scaling by construction)
        wr = WORKLOADS["hrot"]()
        wr.setup(lib, torch, rank, world, False)
        for _ in range(10):
            wr.step()
        rsteps = max(5, min(args.steps, 400))
        rms = time_blocks(torch, dist, world, wr, rsteps, 1, barrier)[0]
        side["replicas"] = {"value": world * rsteps / (rms / 1e3), "unit": wl.unit, "scaling": "weak",
                            "parallelism": "independent ciphertexts per GPU, no collective"}
        del wr
        torch.cuda.empty_cache()

    # end to end: pinned host buffers in and out through the same C ABI calls, three streams
    dog.at("end to end")
    e2e_steps = max(5, min(args.steps, 200))
    for _ in range(3):
        wl.e2e_step()
    wl.e2e_drain()
    barrier()
    t0 = time.perf_counter()
    h2d = d2h = 0
    for _ in range(e2e_steps):
        h2d, d2h = wl.e2e_step()
    wl.e2e_drain()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    # the copies alone: the same bytes up and down per step on two streams, nothing computed
    pipe = wl.pipe
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        slot = i % pipe.depth
        with torch.cuda.stream(pipe.s_in):
            for d, h in zip(pipe.dev_in[slot], pipe.last_host_ins):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(pipe.s_out):
            for h, d in zip(pipe.host_out[slot], pipe.dev_out[slot]):
                h.copy_(d, non_blocking=True)
    torch.cuda.synchronize()
    copy_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s, copy_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, copy_s = float(t[0].item()), float(t[1].item())

    dog.at("report")
    if rank == 0:
        latency = getattr(wl, "latency_metric", False)
        value = ms / args.steps if latency else job_ops * ops * args.steps / (ms / 1e3)
        per_step = sorted(b / args.steps for b in block_ms)
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": not latency,
            "scaling": "strong" if sharded else "weak",
            "vs_baseline": None, "dtype": getattr(wl, "dtype", "u64"), "data": "synthetic",
            "config": {"workload": wl.name},
            "verified": verified,
            "l2": "working set larger than L2 (keys + ciphertexts + workspace > 126 MB)",
            "inflight": getattr(wl, "inflight", 1),
            "parallelism": ("single GPU" if world == 1 else
                            "every ciphertext and key limb-sharded over %d ranks (%s extension limbs), NCCL all-gather "
                            "where limbs must meet, %d operations in flight" % (world, args.ext, wl.inflight)
                            if sharded and args.workload == "hrot" else
                            "the program as the reference's compiler partitioned it over %d GPUs, one process per partition, "
                            "drm / ags / ard records on NCCL" % world if sharded
                            else "independent ciphertexts per GPU"),
            "repeat": {"blocks": len(block_ms), "steps_per_block": args.steps, "ms_per_step_median": per_step[len(per_step) // 2],
                       "ms_per_step_min": per_step[0], "ms_per_step_max": per_step[-1]},
            "e2e": {"value": (1e3 * e2e_s / e2e_steps if latency else job_ops * ops * e2e_steps / e2e_s), "unit": wl.unit,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "copy_ceiling": (1e3 * copy_s / e2e_steps if latency else job_ops * ops * e2e_steps / copy_s),
                    "copy_ceiling_note": "the same bytes up and down per step with nothing computed, same streams and buffers",
                    "numa_node": numa},
            "gpu_launches": wl.gpu_launches_per_step * args.steps,
            "roofline": roofline,
            # the 64-bit transforms are also bound by arithmetic: butterflies per second of the same launch
            # pair against the register-only rate of the butterfly these primes use (FP64 pipe for primes
            # below 2^50), measured on this GPU just now
            "arith_roofline": ({"pipe": "int32", "achieved_gbutterfly_s": rl_limbs * (N // 2) * 16 / (rl_ms / 1e3) / 1e9,
                                "peak_gbutterfly_s": probe["butterfly_u32"], "probe": probe}
                               if getattr(wl, "dtype", "u64") == "u32" else
                               {"pipe": "fp64", "achieved_gbutterfly_s": rl_limbs * (N // 2) * 16 / (rl_ms / 1e3) / 1e9,
                                "peak_gbutterfly_s": probe["butterfly_u64_fp64"], "probe": probe}),
            "step_algorithmic_gbs": job_ops * wl.alg_bytes * args.steps / (ms / 1e3) / 1e9,
            "clocks": clocks,
        }
        line["arith_roofline"]["frac"] = (line["arith_roofline"]["achieved_gbutterfly_s"]
                                          / line["arith_roofline"]["peak_gbutterfly_s"])
        line.update(side)
        if hasattr(wl, "precision_bits"):
            line["precision_bits"] = wl.precision_bits
            line["verified_by"] = "decryption: the output ciphertext against the input slots (bootstrap_runner.py:159-170)"
        if world == 1 and args.workload == "hrot" and not args.no_sub:
            line["sub"] = {name: sub_measurement(torch, lib, name, 200, peak, peak_kind, oracle) for name in ("hmult", "ntt")}
        if not args.no_cpu_baseline and world == 1:
            import oracle
            oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
            v, sample = wl.cpu_sample(oracle)
            line["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
                                    "port_quality": PORT_QUALITY, "sample": sample}
        print(json.dumps(line), flush=True)
    dog.at("shutdown")
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()
    dog.done = True


if __name__ == "__main__":
    main()
