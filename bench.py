"""Benchmark of the BPE training / trie-encoding hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config 3]

Default workload (config 3 of the benchmark list): train 32,000 merges on 1 GiB of seeded synthetic
UTF-8 text.  One step = one complete training run on the HBM-resident corpus: re-tag the symbols,
then the whole merge loop (250 CUDA-graph launches of 128 merges, one read-back each).  N > 1 (under
torchrun): the same corpus cut at word starts across the ranks, "fixed" compaction mode, the pair
counts exchanged by this library's kernels over NVLink peer memory (strong scaling).  The merge list
and its counts are compared, all 32,000 entries, with the golden list of tests/golden/.

One JSON line on stdout:
  value        merges/s with the corpus resident in HBM (CUDA events on the library's stream)
  e2e          the same job through the host-buffer entry point b200bpe_train (pinned host input,
               upload, merge loop, merge-list read-back, all inside the timed region)
  roofline     the dominant kernel's algorithmic bytes / its event-timed duration / measured HBM peak
  cpu_baseline the CPU restatement (oracle port) on a bounded sample: the first merges of the same
               corpus, all host cores; `same_sample` is this library's rate on exactly those merges
  encode       config 4: trie encoding of 1 GiB of text in 262,144 documents with the 32,256-entry
               vocabulary of config 3 (GB/s per job, documents sharded across ranks), token ids
               compared with the CPU oracle
`--impl reference` times the CPU restatement alone (the reference itself is browser JavaScript +
WGSL and cannot run on this machine) without loading the CUDA library.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MIB = 1 << 20
METRIC = "train_merges_per_s"
# benchmark configurations: generator kind, seed, corpus bytes, merges
CONFIGS = {1: (1, 1, 1 * MIB, 1000), 2: (2, 2, 64 * MIB, 8000), 3: (2, 3, 1024 * MIB, 32000), 5: (5, 5, 8192 * MIB, 64000)}
ENCODE_SEED, ENCODE_BYTES, ENCODE_DOCS = 4, 1024 * MIB, 262144   # config 4
MARGIN = 1 * MIB   # bytes a rank generates either side of its nominal span to find the word-aligned cuts
# DRAM bytes (read + write) per algorithmic byte, from one ncu capture of each kernel (the summaries
# under profiles/ give the commands): the roofline "traffic" is this ratio times the algorithmic
# bytes of an average launch of the run.
NCU_DRAM_PER_ALGORITHMIC_BYTE = {"pair_count": 1.02, "argmax": 1.00, "merge_compact": 0.93, "trie_walk": 2.03}


def workload_name(cfg: int, nbytes: int, merges: int, seed: int) -> str:
    return (f"config{cfg}: {merges:,} merges on {nbytes // MIB} MiB synthetic UTF-8 (generator kind {CONFIGS[cfg][0]}, seed {seed}); "
            f"one step = reset + the whole merge loop")


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler(threading.Thread):
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.rows, self._stop_evt = index, [], threading.Event()

    def run(self):
        while not self._stop_evt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self._stop_evt.wait(0.2)

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=6)
        sm = [float(r[1]) for r in self.rows if len(r) > 2 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) > 2 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for k, nm in enumerate(names):
                if len(r) > 5 + k and r[5 + k].lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.rows)}


# ── host-only input production (no CUDA library): used by the CPU arm ──
def host_lib():
    S = C.CDLL(os.path.join(ROOT, "gpu_bpe_b200", "libb200bpe_synth.so"))
    S.b200bpe_synth_corpus_range.argtypes = [C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_int]
    S.b200bpe_synth_corpus_range.restype = C.c_int
    S.b200bpe_pretokenize.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p]
    S.b200bpe_pretokenize.restype = C.c_int
    return S


def host_corpus_prefix(cfg: int, nbytes: int):
    """The first nbytes of the configuration's corpus and their word-start mask, made on the host cores."""
    kind, seed, total, _ = CONFIGS[cfg]
    S = host_lib()
    data = np.empty(nbytes, np.uint8)
    assert S.b200bpe_synth_corpus_range(kind, seed, total, 0, nbytes, data.ctypes.data, os.cpu_count() or 1) == 0
    mask = np.empty(nbytes, np.uint8)
    lo = 0
    while lo < nbytes:   # slices that end after a newline: the boundary rules restart there, and the slices bound the memory
        hi = min(nbytes, lo + 128 * MIB)
        if hi < nbytes:
            hi = lo + int(np.flatnonzero(data[lo:hi] == 0x0A)[-1]) + 1
        assert S.b200bpe_pretokenize(data[lo:hi].ctypes.data, hi - lo, mask[lo:hi].ctypes.data) == 0
        lo = hi
    return data, mask


def available_host_gib() -> float:
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) / (1 << 20)
    except Exception:
        pass
    return 0.0


_CPU_INPUT = {}   # configuration → (symbols, bytes used): the CPU arm builds its input once, outside its timed steps


def cpu_sample(cfg: int, mode: str, seconds: float, max_merges: int):
    """The oracle port on the first merges of the configuration's corpus, all host cores, bounded by
    `seconds`.  The whole corpus is used when the host has the memory for it (u32 symbols, two
    buffers), else a prefix of it, which the sample text then says."""
    from oracle import cpu_oracle as O
    kind, seed, total, _ = CONFIGS[cfg]
    if cfg not in _CPU_INPUT:
        nbytes = total
        while nbytes > 64 * MIB and available_host_gib() < 14.0 * nbytes / (1 << 30) + 4.0:
            nbytes //= 2
        data, mask = host_corpus_prefix(cfg, nbytes)
        _CPU_INPUT[cfg] = (data.astype(np.uint32) | (mask.astype(np.uint32) << 16), nbytes)
        del data, mask
    sym, nbytes = _CPU_INPUT[cfg]
    cores = os.cpu_count() or 1
    r = O.train(sym, max_merges, mode, threads=cores, max_seconds=seconds, want_symbols=False)
    done = int(r["merges"].shape[0])
    what = "the whole corpus" if nbytes == total else f"the first {nbytes // MIB} MiB of the corpus (host memory)"
    return {"value": done / r["seconds"] if r["seconds"] > 0 else 0.0, "unit": "merges/s", "cores": cores, "kind": "port",
            "merges": done, "corpus_bytes": nbytes,
            "sample": f"first {done} merges on {what} ({r['seconds']:.1f} s; these are the most expensive merges of the "
                      f"job: the corpus shrinks as merges are applied)"}, r


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, seed, nbytes, merges = CONFIGS[args.config]
    merges = args.merges or merges
    mode = args.mode or "fixed"
    times, vals, base = [], [], None
    # every step is a bounded sample; the bound shrinks with the number of steps so that the whole
    # command stays within a few minutes
    per_step = min(args.ref_seconds, max(2.0, 200.0 / max(1, args.warmup + args.steps)))
    for i in range(args.warmup + args.steps):
        base, r = cpu_sample(args.config, mode, per_step, args.ref_merges)
        if i >= args.warmup:
            times.append(r["seconds"] * 1e3)
            vals.append(base["value"])
    v = float(np.mean(vals)) if vals else 0.0
    base["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "merges/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": float(np.mean(times)) if times else None, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": workload_name(args.config, nbytes, merges, seed), "compat_mode": mode, "merges": merges,
                   "symbols": nbytes},
        "note": "each step is a time-bounded sample of the merge loop on the host cores (the first merges of the job)",
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": "merges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def golden_merges(cfg: int, mode: str):
    p = os.path.join(ROOT, "tests", "golden", f"config{cfg}_{mode}.npz")
    if not os.path.exists(p):
        return None
    g = np.load(p)
    return np.stack([g["a"].astype(np.uint32), g["b"].astype(np.uint32), g["count"].astype(np.uint32)], axis=1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--config", type=int, default=3, choices=sorted(CONFIGS), help="benchmark configuration (default 3)")
    ap.add_argument("--merges", type=int, default=0, help="for experiments only: fewer merges than the configuration's")
    ap.add_argument("--mode", default=None, help="literal | fixed (default fixed: the mode every GPU count can run)")
    ap.add_argument("--ref-seconds", type=float, default=10.0, help="CPU arm: time bound of one step")
    ap.add_argument("--ref-merges", type=int, default=64, help="CPU arm: most merges of one step")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--e2e-runs", type=int, default=3)
    ap.add_argument("--no-encode", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-profile", action="store_true", help="skip the extra run that times every kernel")
    ap.add_argument("--nccl-exchange", action="store_true", help="sharded runs: NCCL exchange instead of peer memory")
    ap.add_argument("--corpus-mib", type=int, default=0, help="for profiler captures only: the first MiB of the configuration's corpus")
    ap.add_argument("--encode-mib", type=int, default=0, help="for profiler captures only: encode this many MiB instead of config 4's 1024")
    ap.add_argument("--budget-seconds", type=float, default=780.0,
                    help="wall-clock budget of the whole command: the parts after the timed steps are shortened or left out "
                         "(and named under \"skipped\") when they would not fit")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    from gpu_bpe_b200 import BPEEngine, TrainerSession, TrieTokenizer, _lib, synth
    from gpu_bpe_b200.sharding import document_cuts
    from gpu_bpe_b200.vocab import Vocab

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N > 1 with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mode = args.mode or "fixed"
    kind, seed, nbytes, cfg_merges = CONFIGS[args.config]
    full_corpus = not args.corpus_mib or args.corpus_mib * MIB >= nbytes
    if not full_corpus:
        nbytes = args.corpus_mib * MIB   # the generator is prefix-stable only per call: this is a different, smaller corpus
    n_goal = args.merges or cfg_merges
    L = _lib.lib()
    t_begin = time.perf_counter()
    skipped = []

    def seconds_left() -> float:
        return args.budget_seconds - (time.perf_counter() - t_begin)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: int) -> int:
        if world == 1:
            return int(x)
        t = torch.tensor([x], dtype=torch.int64, device="cuda")
        dist.all_reduce(t)
        return int(t.item())

    engine = BPEEngine(local)
    if world > 1:
        uid = [BPEEngine.make_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        engine.init_distributed(rank, world, uid[0])
    else:
        engine.init()

    # ── inputs: every rank makes only its own span of the seeded corpus (plus a margin either side) and
    # pre-tokenises it on its GPU; the cut between two ranks is the first word start at or after r * n / world,
    # which both neighbours find in their margins ──
    lo_nom, hi_nom = nbytes * rank // world, nbytes * (rank + 1) // world
    g_lo, g_hi = max(0, lo_nom - MARGIN), min(nbytes, hi_nom + MARGIN)
    t0 = time.perf_counter()
    gen = synth.corpus_range(kind, seed, nbytes, g_lo, g_hi - g_lo)
    start = 0
    if g_lo > 0:   # the boundary rules restart after a newline
        start = int(np.flatnonzero(gen[:MARGIN // 2] == 0x0A)[0]) + 1
    d_gen = torch.from_numpy(gen[start:]).cuda()
    d_gmask = torch.empty(d_gen.numel(), dtype=torch.uint8, device="cuda")
    pt_ms = []
    for _ in range(3):   # the call synchronises before it returns
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        _lib.check(L.b200bpe_pretokenize_device(engine.ctx, C.c_void_p(d_gen.data_ptr()), d_gen.numel(), C.c_void_p(d_gmask.data_ptr())),
                   "b200bpe_pretokenize_device")
        pt_ms.append((time.perf_counter() - t1) * 1e3)
    pretok = {"device_GB_per_s": d_gen.numel() / 1e9 / (min(pt_ms) / 1e3), "device_ms": min(pt_ms), "bytes": int(d_gen.numel()),
              "what": "word-start mask of this rank's span on its GPU (b200bpe_pretokenize_device), host wall time of the call"}

    def first_start_at_or_after(pos_abs: int) -> int:
        i = pos_abs - (g_lo + start)
        win = d_gmask[i:i + MARGIN // 2]
        nz = torch.nonzero(win)
        assert nz.numel() > 0, "no word start near a shard boundary"
        return i + int(nz[0].item())

    c_lo = 0 if rank == 0 else first_start_at_or_after(lo_nom)
    c_hi = d_gen.numel() if rank == world - 1 else first_start_at_or_after(hi_nom)
    d_bytes = d_gen[c_lo:c_hi].clone()
    d_mask = d_gmask[c_lo:c_hi].clone()
    my_n = c_hi - c_lo
    my_data = gen[start + c_lo:start + c_hi]
    del d_gen, d_gmask
    torch.cuda.empty_cache()
    setup_s = time.perf_counter() - t0
    assert sum_over_ranks(my_n) == nbytes, "the shards do not add up to the corpus"
    flush = torch.empty(256 * MIB, dtype=torch.uint8, device="cuda")  # > L2, rewritten between steps

    flags = _lib.FLAG_NCCL_EXCHANGE if args.nccl_exchange else 0
    sess = TrainerSession.create(engine, d_bytes.data_ptr(), d_mask.data_ptr(), n=my_n, device_pointers=True,
                                 target_vocab_size=256 + n_goal, compat_mode=mode, flags=flags)
    exchange = sess.exchange_kind()
    step_ms, merges, counts = [], None, None
    sampler = None
    launches_before = 0
    for i in range(args.warmup + args.steps):
        flush.fill_(i & 0xFF)
        barrier()
        if i == args.warmup:
            sampler = ClockSampler(local)
            sampler.start()
            launches_before = sess.launches()
        sess.reset()
        merges, counts, early = sess.run()
        torch.cuda.synchronize()
        ms = max_over_ranks(sess.last_reset_ms() + sess.last_run_ms())
        barrier()
        if i >= args.warmup:
            step_ms.append(ms)
    clocks = sampler.stop() if sampler else {}
    gpu_launches = (sess.launches() - launches_before) * world
    n_merges = int(merges.shape[0])
    ms_per_step = float(np.mean(step_ms))
    value = n_merges / (ms_per_step / 1e3)
    batches = (n_merges + 127) // 128

    # ── parity: the whole merge list and its counts against the golden list of the configuration ──
    parity = {"config": args.config, "mode": mode, "merges_compared": 0, "against": None}
    gold = golden_merges(args.config, mode) if full_corpus else None
    if gold is not None:
        k = min(n_merges, gold.shape[0])
        assert k == min(n_goal, gold.shape[0]), f"the run stopped after {n_merges} merges, the golden list has {gold.shape[0]}"
        got = np.stack([merges[:k, 0], merges[:k, 1], counts[:k]], axis=1)
        bad = np.flatnonzero((got != gold[:k]).any(axis=1))
        assert bad.size == 0, f"merge {int(bad[0])} differs from the golden list: got {got[bad[0]].tolist()}, want {gold[bad[0]].tolist()}"
        assert np.array_equal(merges[:k, 2], 256 + np.arange(k)), "new ids are not consecutive"
        parity.update(merges_compared=k, against=f"tests/golden/config{args.config}_{mode}.npz (pairs and counts, bit-exact)")
    if world > 1:   # every rank holds the same list
        h = int(np.bitwise_xor.reduce((merges.astype(np.uint64) * np.arange(1, 4, dtype=np.uint64)).ravel())) & ((1 << 62) - 1)
        t = torch.tensor([h, -h], dtype=torch.int64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert int(t[0].item()) == h and int(t[1].item()) == -h, "ranks disagree on the merge list"
        parity["ranks_agree"] = True

    # ── per-kernel device time: one more run with every kernel bracketed by CUDA events ──
    peak, peak_src = measured_hbm_peak()
    roofline = None
    step_s = ms_per_step / 1e3
    e2e_runs = args.e2e_runs
    # what is still to come, in seconds: the end-to-end runs (the headline) are kept before everything else
    need_e2e = lambda runs: (1 if runs > 0 else 0) * (1.15 * step_s + 2) + max(1, runs) * (1.15 * step_s + 2)
    while e2e_runs > 0 and need_e2e(e2e_runs) > seconds_left() - 20:
        e2e_runs -= 1
    if e2e_runs != args.e2e_runs:
        skipped.append(f"e2e runs cut from {args.e2e_runs} to {max(1, e2e_runs)}{'' if e2e_runs else ' (no untimed run before it)'}")
    do_profile = not args.no_profile and (1.6 * step_s + 5) < seconds_left() - need_e2e(e2e_runs) - 20
    if world > 1:   # every rank takes the same decisions
        t = torch.tensor([e2e_runs, int(do_profile)], dtype=torch.int64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        e2e_runs, do_profile = int(t[0].item()), bool(t[1].item())
    if not args.no_profile and not do_profile:
        skipped.append("per-kernel timing run (roofline)")
    if do_profile:
        prof = TrainerSession.create(engine, d_bytes.data_ptr(), d_mask.data_ptr(), n=my_n, device_pointers=True,
                                     target_vocab_size=256 + n_goal, compat_mode=mode, flags=flags | _lib.FLAG_TIME_KERNELS)
        barrier()
        prof.run()
        ks = prof.kernel_stats()
        prof.destroy()
        kern = {}
        for name in ("pair_count", "argmax", "merge_compact"):
            ms_tot, launches, nb = ks[f"{name}_ms"], ks[f"{name}_launches"], ks[f"{name}_bytes"]
            gbs = (nb / 1e9) / (ms_tot / 1e3) if ms_tot > 0 else 0.0
            kern[name] = {"ms_total": ms_tot, "launches": launches, "avg_us": 1e3 * ms_tot / max(1, launches),
                          "algorithmic_GB": nb / 1e9, "achieved_GBps": gbs, "frac_of_peak": gbs / peak}
        kern["pair_count"]["skipped_launches"] = ks["pair_count_skipped_launches"]
        kern["pair_count"]["skipped_ms_total"] = ks["pair_count_skipped_ms"]
        if world > 1:
            kern["exchange"] = {"ms_total": ks["exchange_ms"], "launches": ks["exchange_launches"],
                                "avg_us": 1e3 * ks["exchange_ms"] / max(1, ks["exchange_launches"]), "kind": exchange}
        dom = max(("pair_count", "argmax", "merge_compact"), key=lambda k: kern[k]["ms_total"])
        roofline = {"bound": "hbm", "kernel": "k_" + dom, "achieved": kern[dom]["achieved_GBps"], "peak": peak, "unit": "GB/s",
                    "frac": kern[dom]["frac_of_peak"], "peak_source": peak_src,
                    "traffic": NCU_DRAM_PER_ALGORITHMIC_BYTE[dom] * kern[dom]["algorithmic_GB"] * 1e9 / max(1, kern[dom]["launches"]),
                    "traffic_how": "DRAM read + write bytes per launch: the ncu ratio of DRAM to algorithmic bytes for this kernel "
                                   "(one capture, summary under profiles/) x the algorithmic bytes of an average launch",
                    "per_launch_algorithmic_bytes": kern[dom]["algorithmic_GB"] * 1e9 / max(1, kern[dom]["launches"]),
                    "avg_launch_us": kern[dom]["avg_us"], "kernels": kern,
                    "how": "one extra run with CUDA events around every kernel on the library's stream (no graph), this rank"}

    # ── end to end: host buffers through b200bpe_train, upload and read-back inside the timed region ──
    pin_b = torch.from_numpy(my_data.copy()).pin_memory()
    pin_m = d_mask.cpu().pin_memory()
    opts = TrainerSession._opts(256 + n_goal, 256, mode, 128, 0, flags)
    out = np.zeros((n_goal, 3), np.uint32)
    cnt = np.zeros(n_goal, np.uint32)
    e2e_ms = []
    e2e_warm = 1 if e2e_runs > 0 else 0   # 0 runs asked for (or left by the budget): one timed run with no untimed one before it
    for i in range(e2e_warm + max(1, e2e_runs)):
        flush.fill_(i & 0xFF)
        barrier()
        nm, es = C.c_uint32(), C.c_uint32()
        t0 = time.perf_counter()
        st = L.b200bpe_train(engine.ctx, C.c_void_p(pin_b.data_ptr()), C.c_void_p(pin_m.data_ptr()), my_n,
                             C.byref(opts), out.ctypes.data_as(_lib.u32p), cnt.ctypes.data_as(_lib.u32p),
                             C.byref(nm), C.byref(es), _lib.PROGRESS_CB(), None)
        _lib.check(st, "b200bpe_train")
        torch.cuda.synchronize()
        dt = max_over_ranks((time.perf_counter() - t0) * 1e3)
        barrier()
        if i >= e2e_warm:
            e2e_ms.append(dt)
        assert np.array_equal(out[: nm.value], merges), "host-buffer run and resident run disagree"
    e2e_step = float(np.median(e2e_ms))
    e2e = {"value": n_merges / (e2e_step / 1e3), "unit": "merges/s", "ms_per_step": e2e_step,
           "h2d_bytes_per_step": int(2 * my_n), "d2h_bytes_per_step": int(n_merges * 16 + batches * 224),
           "ms_samples": [round(x, 1) for x in e2e_ms],
           "api": "b200bpe_train (host bytes + word-start mask in pinned memory → merge list), per rank"}
    del pin_b, pin_m

    # ── the CPU restatement on a bounded sample, and this library on exactly the same merges ──
    cpu = None
    do_cpu = not args.no_cpu and seconds_left() > 3 * args.cpu_seconds + 60
    if not args.no_cpu and not do_cpu:
        skipped.append("cpu_baseline sample")
    if rank == 0 and world == 1 and do_cpu:
        cpu, r = cpu_sample(args.config, mode, args.cpu_seconds, args.ref_merges)
        _CPU_INPUT.clear()
        k = cpu["merges"]
        if cpu["corpus_bytes"] == nbytes:
            assert np.array_equal(r["merges"][:, :3], merges[:k]) and np.array_equal(r["merges"][:, 3], counts[:k]), \
                "the CPU oracle's first merges differ from the GPU's"
            cpu["checked"] = f"the oracle's {k} merges and counts equal the GPU's first {k}"
            sess.reset()
            sess.run(k)
            same_ms = sess.last_run_ms()
            cpu["same_sample"] = {"gpu_merges_per_s": k / (same_ms / 1e3), "gpu_ms": same_ms,
                                  "ratio": (k / (same_ms / 1e3)) / cpu["value"] if cpu["value"] else None,
                                  "what": f"this library (resident corpus, one GPU) on the same first {k} merges"}
    sess.destroy()
    del d_bytes, d_mask, flush
    torch.cuda.empty_cache()

    # ── encode (config 4): documents sharded across ranks, no collective ──
    encode = None
    do_encode = not args.no_encode and seconds_left() > 90
    if world > 1:
        t = torch.tensor([int(do_encode)], dtype=torch.int64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        do_encode = bool(t[0].item())
    if not args.no_encode and not do_encode:
        skipped.append("encode (config 4)")
    enc_bytes = args.encode_mib * MIB if args.encode_mib else ENCODE_BYTES
    enc_docs = max(1, ENCODE_DOCS * enc_bytes // ENCODE_BYTES)
    if do_encode:
        gold3 = golden_merges(3, "fixed")
        if args.config == 3 and n_merges == 32000:
            vm = merges
        elif gold3 is not None:
            vm = gold3
        else:
            vm = merges
        vocab = Vocab()
        for a, b in vm[:, :2].tolist():
            vocab.addMerge(a, b)
        tok = TrieTokenizer.fromVocab(engine, vocab.entries)
        sub, lg = C.c_uint32(), C.c_uint32()
        L.b200bpe_tokenizer_layout(tok._h, C.byref(sub), C.byref(lg))
        offs = synth.doc_offsets(ENCODE_SEED, enc_bytes, enc_docs, 1.0)
        dcut = document_cuts(offs, world)
        d0, d1 = int(dcut[rank]), int(dcut[rank + 1])
        b0, b1 = int(offs[d0]), int(offs[d1])
        my_text = synth.corpus_range(2, ENCODE_SEED, enc_bytes, b0, b1 - b0)
        my_offs = (offs[d0:d1 + 1] - offs[d0]).astype(np.uint64)
        d_text = torch.from_numpy(my_text).cuda()
        d_offs = torch.from_numpy(my_offs.view(np.int64).copy()).cuda()
        d_tok = torch.empty(max(1, b1 - b0), dtype=torch.int32, device="cuda")
        d_toff = torch.empty(d1 - d0 + 1, dtype=torch.int64, device="cuda")
        flush = torch.empty(256 * MIB, dtype=torch.uint8, device="cuda")
        enc_ms, walk_ms, comp_ms, ntok = [], [], [], 0
        for i in range(3 + 5):
            flush.fill_(i & 0xFF)
            barrier()
            ntok = tok.encodeBatchDevice(d_text.data_ptr(), d_offs.data_ptr(), d1 - d0, b1 - b0, d_tok.data_ptr(),
                                         d_tok.numel(), d_toff.data_ptr())
            w, c = tok.lastKernelMs()
            t = max_over_ranks(w + c)
            if i >= 3:
                enc_ms.append(t); walk_ms.append(w); comp_ms.append(c)
        # end to end through b200bpe_encode_batch with pinned host buffers owned by the caller:
        # upload, the kernels, read-back of the offsets and of exactly the tokens produced
        pin_t = torch.from_numpy(my_text).pin_memory()
        pin_out = torch.empty(max(1, b1 - b0), dtype=torch.int32).pin_memory()
        toff_h = np.zeros(d1 - d0 + 1, np.uint64)
        e_ms = []
        for i in range(3):
            barrier()
            t0 = time.perf_counter()
            st = L.b200bpe_encode_batch(tok._h, C.c_void_p(pin_t.data_ptr()), my_offs.ctypes.data, d1 - d0,
                                        C.c_void_p(pin_out.data_ptr()), pin_out.numel(), toff_h.ctypes.data)
            _lib.check(st, "b200bpe_encode_batch")
            e_ms.append(max_over_ranks((time.perf_counter() - t0) * 1e3))
        assert int(toff_h[-1]) == ntok, "host-buffer encode and resident encode disagree on the token count"
        got_tok = pin_out[:ntok].numpy().view(np.uint32)
        assert torch.equal(pin_out[:ntok], d_tok[:ntok].cpu()), "host-buffer encode and resident encode disagree on the tokens"
        assert np.array_equal(toff_h.astype(np.int64), d_toff.cpu().numpy()), "document token offsets disagree"
        # token ids against the CPU oracle, every document of this rank (outside every timed region)
        enc_parity = None
        if not args.no_cpu:
            from oracle import cpu_oracle as O
            from oracle import wgsl_model as M
            trie = M.compile_vocab_to_trie(vocab.entries)
            want_tok, want_off = O.encode_batch(my_text, my_offs, trie, tok.chunkSize, threads=max(1, (os.cpu_count() or 1) // world))
            ok = want_tok.size == ntok and np.array_equal(want_tok, got_tok) and np.array_equal(want_off, toff_h)
            assert sum_over_ranks(0 if ok else 1) == 0, "token ids differ from the CPU oracle"
            enc_parity = "every token id and document offset equal to the CPU oracle's (all documents, all ranks)"
        e_ms = e_ms[1:]
        tot_tok = sum_over_ranks(ntok)
        w_ms, c_ms = float(np.mean(walk_ms)), float(np.mean(comp_ms))
        alg_bytes = (b1 - b0) + 4 * ntok
        encode = {"metric": "encode_GB_per_s", "value": enc_bytes / 1e9 / (float(np.mean(enc_ms)) / 1e3), "unit": "GB/s",
                  "workload": f"config4: {enc_bytes // MIB} MiB synthetic UTF-8 (seed {ENCODE_SEED}) in {enc_docs} lognormal documents, "
                              f"{len(vocab.entries)}-entry vocabulary (the merge list of config 3), chunk {tok.chunkSize}",
                  "trie": {"nodes": tok.nodeCount, "edges": tok.edgeCount, "max_token_len": tok.maxTokenLen,
                           "layout": {0: "global hash table behind a probe cache", 1: "hybrid: hot transitions in shared memory, two-byte first step"}.get(sub.value, "shared-memory cuckoo table"),
                           "log2_slots": lg.value},
                  "tokens": tot_tok, "walk_ms": w_ms, "scan_compact_ms": c_ms, "scaling": "strong",
                  "e2e_GB_per_s": enc_bytes / 1e9 / (float(np.mean(e_ms)) / 1e3),
                  "e2e_h2d_bytes": int(b1 - b0 + 8 * (d1 - d0 + 1)), "e2e_d2h_bytes": int(4 * ntok + 8 * (d1 - d0 + 1)),
                  "parity": enc_parity,
                  "roofline": {"bound": "hbm", "kernel": "k_trie_walk", "achieved": alg_bytes / 1e9 / (w_ms / 1e3),
                               "peak": peak, "unit": "GB/s", "frac": alg_bytes / 1e9 / (w_ms / 1e3) / peak,
                               "traffic": NCU_DRAM_PER_ALGORITHMIC_BYTE["trie_walk"] * alg_bytes,
                               "algorithmic_bytes": "L input bytes + 4 T token bytes (this rank)"}}
        tok.destroy()

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "merges/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": {"workload": workload_name(args.config, nbytes, n_goal, seed), "compat_mode": mode, "merges": n_goal,
                       "symbols": nbytes},
            "parallelism": "single GPU" if world == 1 else f"corpus cut at word starts over {world} GPUs, {exchange} count exchange",
            "l2": f"inputs ({4 * nbytes // world // MIB} MiB of symbols per buffer and rank) exceed L2; a 256 MiB buffer is rewritten between steps",
            "setup_s": setup_s, "e2e": e2e, "gpu_launches": int(gpu_launches), "clocks": clocks, "roofline": roofline,
            "cpu_baseline": cpu, "encode": encode, "pretokenize": pretok, "parity": parity, "skipped": skipped,
        }))
    if world > 1:
        dist.destroy_process_group()
    engine.destroy()


if __name__ == "__main__":
    main()
