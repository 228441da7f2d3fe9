"""Benchmark of the BPE training / trie-encoding hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1 workload: train 8,000 merges on 64 MiB of seeded synthetic UTF-8 text (the second benchmark
configuration); one step = one complete training run (re-tag the resident corpus, run the merge
loop).  N > 1 (under torchrun): the same corpus cut at word starts across the ranks, "fixed"
compaction mode, one NCCL count exchange + one 32-byte all-reduce per merge (strong scaling).

One JSON line on stdout:
  value        merges/s with the corpus resident in HBM (CUDA events on the library's stream)
  e2e          the same job through the host-buffer entry point b200bpe_train (pinned host input,
               upload, merge loop, merge-list read-back, all inside the timed region)
  roofline     the dominant kernel's algorithmic bytes / its event-timed duration / measured HBM peak
  cpu_baseline the CPU restatement (oracle port) on a bounded sample, all host cores
  encode       trie encoding of 256 MiB of the same text in 65,536 documents (GB/s), per rank
`--impl reference` times the CPU restatement alone (the reference itself is browser JavaScript +
WGSL and cannot run on this machine).
"""
from __future__ import annotations

import argparse
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
CORPUS_BYTES = 64 * MIB
CORPUS_SEED = 2
MERGES = 8000
ENCODE_BYTES = 256 * MIB
ENCODE_DOCS = 65536
METRIC = "train_merges_per_s"
WORKLOAD = "config2: 8,000 merges on 64 MiB synthetic UTF-8 (seed 2, 50k-word per-script Zipf 1.1 lexicons)"
# DRAM bytes (read + write) per algorithmic byte, from one ncu capture of each kernel (the
# summaries under profiles/ give the commands): the roofline "traffic" is this ratio times the
# algorithmic bytes of an average launch of the run.  Below 1 where the 126 MB L2 keeps part of the
# symbol array from one merge to the next.
NCU_DRAM_PER_ALGORITHMIC_BYTE = {"pair_count": 1.02, "argmax": 1.00, "merge_compact": 0.65, "trie_walk": 1.05}


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


def make_corpus():
    from gpu_bpe_b200 import PreTokenizer, synth
    data = synth.corpus(2, CORPUS_SEED, CORPUS_BYTES)
    mask = PreTokenizer(normalize=False).preTokenizeBytes(data)["wordStarts"]
    return data, mask


def cpu_baseline_sample(data, mask, seconds: float, mode: str):
    """The oracle port on the first merges of the same corpus, all host cores, bounded by `seconds`."""
    from oracle import cpu_oracle as O
    sym = data.astype(np.uint32) | (mask.astype(np.uint32) << 16)
    cores = os.cpu_count() or 1
    r = O.train(sym, MERGES, mode, threads=cores, max_seconds=seconds, want_symbols=False)
    done = int(r["merges"].shape[0])
    return {"value": done / r["seconds"] if r["seconds"] > 0 else 0.0, "unit": "merges/s", "cores": cores,
            "kind": "port",
            "sample": f"first {done} of {MERGES} merges of the 64 MiB corpus ({r['seconds']:.1f} s; later merges "
                      f"are cheaper because the corpus shrinks)"}, r


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    data, mask = make_corpus()
    mode = args.mode or ("literal" if args.gpus == 1 else "fixed")   # the mode the GPU arm runs at this N
    times, vals = [], []
    for i in range(args.warmup + args.steps):
        base, r = cpu_baseline_sample(data, mask, args.ref_seconds, mode)
        if i >= args.warmup:
            times.append(r["seconds"] * 1e3)
            vals.append(base["value"])
    v = float(np.mean(vals)) if vals else 0.0
    base["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "merges/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": float(np.mean(times)) if times else None, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "compat_mode": mode,
                   "note": "each step is a time-bounded sample of the merge loop on the host cores"},
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": "merges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    global MERGES, CORPUS_BYTES, ENCODE_BYTES, ENCODE_DOCS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--ref-seconds", type=float, default=15.0)
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--no-encode", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--merges", type=int, default=MERGES, help="for experiments only; the benchmark is 8,000")
    ap.add_argument("--corpus-mib", type=int, default=CORPUS_BYTES // MIB, help="for experiments only; the benchmark is 64")
    ap.add_argument("--encode-mib", type=int, default=ENCODE_BYTES // MIB, help="for experiments only; the benchmark is 256")
    ap.add_argument("--encode-docs", type=int, default=ENCODE_DOCS, help="for experiments only; the benchmark is 65,536")
    ap.add_argument("--mode", default=None, help="literal | fixed (default: literal on 1 GPU, fixed when sharded)")
    args = ap.parse_args()
    MERGES, CORPUS_BYTES = args.merges, args.corpus_mib * MIB
    ENCODE_BYTES, ENCODE_DOCS = args.encode_mib * MIB, args.encode_docs
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    from gpu_bpe_b200 import BPEEngine, PreTokenizer, TrainerSession, TrieTokenizer, _lib, synth
    from gpu_bpe_b200.sharding import document_cuts, word_aligned_cuts
    from gpu_bpe_b200.vocab import Vocab

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N > 1 with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mode = args.mode or ("literal" if world == 1 else "fixed")

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

    engine = BPEEngine(local)
    if world > 1:
        uid = [BPEEngine.make_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        engine.init_distributed(rank, world, uid[0])
    else:
        engine.init()

    # ── inputs: the whole corpus is generated on every rank (seeded), each keeps its span ──
    data, mask = make_corpus()
    cuts = word_aligned_cuts(mask, world)
    lo, hi = int(cuts[rank]), int(cuts[rank + 1])
    my_data, my_mask = data[lo:hi], mask[lo:hi]
    d_bytes = torch.from_numpy(my_data.copy()).cuda()
    d_mask = torch.from_numpy(my_mask.copy()).cuda()
    flush = torch.empty(256 * MIB, dtype=torch.uint8, device="cuda")  # > L2, rewritten between steps

    sess = TrainerSession.create(engine, d_bytes.data_ptr(), d_mask.data_ptr(), n=hi - lo, device_pointers=True,
                                 target_vocab_size=256 + MERGES, compat_mode=mode)
    step_ms, merges = [], None
    sampler = None
    for i in range(args.warmup + args.steps):
        flush.fill_(i & 0xFF)
        barrier()
        if i == args.warmup:
            sampler = ClockSampler(local)
            sampler.start()
        sess.reset()
        merges, counts, early = sess.run()
        torch.cuda.synchronize()
        ms = max_over_ranks(sess.last_reset_ms() + sess.last_run_ms())
        barrier()
        if i >= args.warmup:
            step_ms.append(ms)
    clocks = sampler.stop() if sampler else {}
    n_merges = int(merges.shape[0])
    ms_per_step = float(np.mean(step_ms))
    value = n_merges / (ms_per_step / 1e3)
    batches = (n_merges + 127) // 128
    # per step: k_tag_symbols; per batch: k_begin_batch, the graph's 128 + 4 spare iterations of
    # {k_pair_count, k_argmax_setup, k_merge_compact} (sharded: + 8 exchange kernels), and k_literal_tail in literal mode
    kernels_per_iter = 3 if world == 1 else 11
    iters = 132 if world == 1 else 128   # sharded runs carry no spare iterations
    gpu_launches = args.steps * (1 + batches * (1 + iters * kernels_per_iter + (1 if mode == "literal" else 0)))

    # ── per-kernel device time: one more run with every kernel bracketed by CUDA events ──
    prof = TrainerSession.create(engine, d_bytes.data_ptr(), d_mask.data_ptr(), n=hi - lo, device_pointers=True,
                                 target_vocab_size=256 + MERGES, compat_mode=mode, flags=_lib.FLAG_TIME_KERNELS)
    prof.run()
    ks = prof.kernel_stats()
    prof.destroy()
    peak, peak_src = measured_hbm_peak()
    kern = {}
    for name in ("pair_count", "argmax", "merge_compact"):
        ms_tot, launches, nbytes = ks[f"{name}_ms"], ks[f"{name}_launches"], ks[f"{name}_bytes"]
        gbs = (nbytes / 1e9) / (ms_tot / 1e3) if ms_tot > 0 else 0.0
        kern[name] = {"ms_total": ms_tot, "launches": launches, "avg_us": 1e3 * ms_tot / max(1, launches),
                      "algorithmic_GB": nbytes / 1e9, "achieved_GBps": gbs, "frac_of_peak": gbs / peak}
    kern["pair_count"]["skipped_launches"] = ks["pair_count_skipped_launches"]
    kern["pair_count"]["skipped_ms_total"] = ks["pair_count_skipped_ms"]
    kern["table_update"] = {"ms_total": ks["table_update_ms"], "launches": ks["merge_compact_launches"],
                            "avg_us": 1e3 * ks["table_update_ms"] / max(1, ks["merge_compact_launches"]),
                            "what": "k_literal_tail (the queued pair deltas are folded in by k_merge_compact itself)"}
    if world > 1:
        kern["exchange"] = {"ms_total": ks["exchange_ms"], "launches": ks["exchange_launches"],
                            "avg_us": 1e3 * ks["exchange_ms"] / max(1, ks["exchange_launches"])}
    dom = max(("pair_count", "argmax", "merge_compact"), key=lambda k: kern[k]["ms_total"])
    roofline = {"bound": "hbm", "kernel": "k_" + dom, "achieved": kern[dom]["achieved_GBps"], "peak": peak, "unit": "GB/s",
                "frac": kern[dom]["frac_of_peak"], "peak_source": peak_src,
                "traffic": NCU_DRAM_PER_ALGORITHMIC_BYTE[dom] * kern[dom]["algorithmic_GB"] * 1e9 / max(1, kern[dom]["launches"]),
                "traffic_how": "DRAM read + write bytes per launch: the ncu ratio of DRAM to algorithmic bytes for this kernel "
                               "(merge 3,000 of this workload for k_merge_compact) x the algorithmic bytes of an average launch",
                "per_launch_algorithmic_bytes": kern[dom]["algorithmic_GB"] * 1e9 / max(1, kern[dom]["launches"]),
                "avg_launch_us": kern[dom]["avg_us"], "kernels": kern,
                "how": "one extra run with CUDA events around every kernel on the library's stream (no graph)"}

    # ── end to end: host buffers through b200bpe_train, upload and read-back inside the timed region ──
    import ctypes as C
    pin_b = torch.from_numpy(my_data.copy()).pin_memory()
    pin_m = torch.from_numpy(my_mask.copy()).pin_memory()
    opts = TrainerSession._opts(256 + MERGES, 256, mode, 128, 0, 0)
    out = np.zeros((MERGES, 3), np.uint32)
    cnt = np.zeros(MERGES, np.uint32)
    e2e_ms = []
    for i in range(2 + max(5, args.steps)):
        flush.fill_(i & 0xFF)
        barrier()
        nm, es = C.c_uint32(), C.c_uint32()
        t0 = time.perf_counter()
        st = _lib.lib().b200bpe_train(engine.ctx, C.c_void_p(pin_b.data_ptr()), C.c_void_p(pin_m.data_ptr()), hi - lo,
                                      C.byref(opts), out.ctypes.data_as(_lib.u32p), cnt.ctypes.data_as(_lib.u32p),
                                      C.byref(nm), C.byref(es), _lib.PROGRESS_CB(), None)
        _lib.check(st, "b200bpe_train")
        torch.cuda.synchronize()
        dt = max_over_ranks((time.perf_counter() - t0) * 1e3)
        barrier()
        if i >= 2:
            e2e_ms.append(dt)
        assert np.array_equal(out[: nm.value], merges), "host-buffer run and resident run disagree"
    e2e_step = float(np.median(e2e_ms))   # of at least five runs: a slow host-side allocation or two do not decide the number
    e2e = {"value": n_merges / (e2e_step / 1e3), "unit": "merges/s", "ms_per_step": e2e_step,
           "h2d_bytes_per_step": int(2 * (hi - lo)), "d2h_bytes_per_step": int(n_merges * 16 + batches * 128),
           "ms_samples": [round(x, 1) for x in e2e_ms],
           "api": "b200bpe_train (host bytes + word-start mask in pinned memory → merge list)"}

    # ── encode: documents sharded across ranks, no collective ──
    encode = None
    if not args.no_encode:
        vocab = Vocab()
        for a, b, _ in merges.tolist():
            vocab.addMerge(a, b)
        tok = TrieTokenizer.fromVocab(engine, vocab.entries)
        text = synth.corpus(2, 4, ENCODE_BYTES)
        offs = synth.doc_offsets(4, ENCODE_BYTES, ENCODE_DOCS, 1.0)
        dcut = document_cuts(offs, world)
        d0, d1 = int(dcut[rank]), int(dcut[rank + 1])
        b0, b1 = int(offs[d0]), int(offs[d1])
        my_text = text[b0:b1]
        my_offs = (offs[d0:d1 + 1] - offs[d0]).astype(np.uint64)
        d_text = torch.from_numpy(my_text.copy()).cuda()
        d_offs = torch.from_numpy(my_offs.view(np.int64).copy()).cuda()
        d_tok = torch.empty(max(1, b1 - b0), dtype=torch.int32, device="cuda")
        d_toff = torch.empty(d1 - d0 + 1, dtype=torch.int64, device="cuda")
        enc_ms, walk_ms, comp_ms, ntok = [], [], [], 0
        for i in range(3 + max(1, args.steps)):
            flush.fill_(i & 0xFF)
            barrier()
            ntok = tok.encodeBatchDevice(d_text.data_ptr(), d_offs.data_ptr(), d1 - d0, b1 - b0, d_tok.data_ptr(),
                                         d_tok.numel(), d_toff.data_ptr())
            w, c = tok.lastKernelMs()
            t = max_over_ranks(w + c)
            if i >= 3:
                enc_ms.append(t); walk_ms.append(w); comp_ms.append(c)
        # end to end through b200bpe_encode_batch with pinned host buffers owned by the caller:
        # upload, both kernels, read-back of the offsets and of exactly the tokens produced
        pin_t = torch.from_numpy(my_text.copy()).pin_memory()
        pin_out = torch.empty(max(1, b1 - b0), dtype=torch.int32).pin_memory()
        toff_h = np.zeros(d1 - d0 + 1, np.uint64)
        e_ms = []
        for i in range(4):
            barrier()
            t0 = time.perf_counter()
            st = _lib.lib().b200bpe_encode_batch(tok._h, C.c_void_p(pin_t.data_ptr()), my_offs.ctypes.data, d1 - d0,
                                                 C.c_void_p(pin_out.data_ptr()), pin_out.numel(), toff_h.ctypes.data)
            _lib.check(st, "b200bpe_encode_batch")
            e_ms.append(max_over_ranks((time.perf_counter() - t0) * 1e3))
        assert int(toff_h[-1]) == ntok, "host-buffer encode and resident encode disagree on the token count"
        assert torch.equal(pin_out[:ntok], d_tok[:ntok].cpu()), "host-buffer encode and resident encode disagree on the tokens"
        assert np.array_equal(toff_h.astype(np.int64), d_toff.cpu().numpy()), "document token offsets disagree"
        e_ms = e_ms[1:]
        tot_tok = ntok
        if world > 1:
            t = torch.tensor([ntok], dtype=torch.int64, device="cuda")
            dist.all_reduce(t)
            tot_tok = int(t.item())
        w_ms, c_ms = float(np.mean(walk_ms)), float(np.mean(comp_ms))
        alg_bytes = (b1 - b0) + 4 * ntok
        encode = {"metric": "encode_GB_per_s", "value": ENCODE_BYTES / 1e9 / (float(np.mean(enc_ms)) / 1e3), "unit": "GB/s",
                  "workload": f"{ENCODE_BYTES // MIB} MiB synthetic UTF-8 in {ENCODE_DOCS} lognormal documents, "
                              f"{256 + n_merges}-entry vocabulary, chunk {tok.chunkSize}",
                  "tokens": tot_tok, "walk_ms": w_ms, "scan_compact_ms": c_ms, "scaling": "strong",
                  "e2e_GB_per_s": ENCODE_BYTES / 1e9 / (float(np.mean(e_ms)) / 1e3),
                  "e2e_h2d_bytes": int(b1 - b0 + 8 * (d1 - d0 + 1)), "e2e_d2h_bytes": int(4 * ntok + 8 * (d1 - d0 + 1)),
                  "roofline": {"bound": "hbm", "kernel": "k_trie_walk", "achieved": alg_bytes / 1e9 / (w_ms / 1e3),
                               "peak": peak, "unit": "GB/s", "frac": alg_bytes / 1e9 / (w_ms / 1e3) / peak,
                               "traffic": NCU_DRAM_PER_ALGORITHMIC_BYTE["trie_walk"] * alg_bytes,
                               "algorithmic_bytes": "L input bytes + 4 T token bytes (this rank)"}}
        tok.destroy()

    # ── pre-tokeniser on the device (a "next" row beside the hot path): word starts of this rank's bytes ──
    pretok = None
    if not args.no_encode:
        import ctypes as C
        d_ws = torch.empty(hi - lo, dtype=torch.uint8, device="cuda")
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        pt_ms = []
        for i in range(4):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            _lib.check(_lib.lib().b200bpe_pretokenize_device(engine.ctx, C.c_void_p(d_bytes.data_ptr()), hi - lo,
                                                              C.c_void_p(d_ws.data_ptr())), "b200bpe_pretokenize_device")
            pt_ms.append((time.perf_counter() - t0) * 1e3)   # the call synchronises before it returns
        assert np.array_equal(d_ws.cpu().numpy(), my_mask), "device pre-tokeniser and host pre-tokeniser disagree"
        sample = my_data[: 8 * MIB]
        t0 = time.perf_counter()
        PreTokenizer(normalize=False).preTokenizeBytes(sample)
        host_s = time.perf_counter() - t0
        pretok = {"device_GB_per_s": (hi - lo) / 1e9 / (min(pt_ms[1:]) / 1e3), "device_ms": min(pt_ms[1:]),
                  "host_GB_per_s": sample.size / 1e9 / host_s, "host_sample": "first 8 MiB, one core",
                  "checked": "word-start mask identical to the host pre-tokeniser on the whole corpus"}

    cpu = None
    parity = None
    if rank == 0 and not args.no_cpu:
        # N = 1: the timed CPU baseline; N > 1: a shorter run of the same oracle, only as the checker
        sample, r = cpu_baseline_sample(data, mask, args.cpu_seconds if world == 1 else min(args.cpu_seconds, 6.0), mode)
        k = int(r["merges"].shape[0])
        assert np.array_equal(r["merges"][:, :3], merges[:k]), "GPU merge list differs from the CPU oracle"
        assert np.array_equal(r["merges"][:, 3], counts[:k]), "GPU pair counts differ from the CPU oracle"
        parity = f"first {k} merges and their counts bit-exact with the CPU oracle"
        if world == 1:
            cpu = sample
            cpu["checked"] = parity

    sess.destroy()
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "merges/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "compat_mode": mode, "merges": n_merges, "symbols": int(data.size),
                       "l2": "inputs (256 MiB of symbols per buffer) exceed L2; a 256 MiB buffer is rewritten between steps",
                       "parallelism": "single GPU" if world == 1 else f"corpus cut at word starts over {world} GPUs"},
            "e2e": e2e, "gpu_launches": gpu_launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "encode": encode, "pretokenize": pretok, "parity": parity,
        }))
    if world > 1:
        dist.destroy_process_group()
    engine.destroy()


if __name__ == "__main__":
    main()
